"""The allocation-free matmul entry (`jq_matmul_t_dev_noalloc`) against the ordinary device entry.

Some callers cannot let this library allocate: the GPU's memory is already fully assigned by the host
application, or the call sits in a loop where a cudaMalloc (driver lock, possible device synchronisation) is
not tolerable.  For them the library carries its scratch - the int8 activation planes passed between the
two kernels of a decode product - in a fixed 4 MiB device array.  The test calls the entry through the C ABI
twice in a row with different inputs (the array keeps the first call's contents, so the second call shows
that stale data is not read) and compares with `jq_matmul_t_dev`, which takes its planes in shared memory or
in allocated scratch, and with the CPU oracle.  It also checks the property the entry exists for: once the
first call on the device has done its set-up, a call leaves the amount of free device memory unchanged.
This file is collected last, so a failure here cannot hide another test's result.
"""
import ctypes

import numpy as np
import pytest

import oracle
from joshua_b200 import _lib, synth
from joshua_b200._lib import JoshuaB200Error, check
from joshua_b200.qtensor import QTensor
from tests.gpu_util import TOL, assert_close

pytestmark = pytest.mark.gpu


def noalloc(q, mkn, x, y):
    import torch

    m, k, n = mkn
    check(_lib.lib().jq_matmul_t_dev_noalloc(q._h, m, k, n, x.data_ptr(), y.data_ptr(),
                                             torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("type_id,mkn", [(synth.Q4_K, (1, 4096, 1024)), (synth.Q4_K, (8, 14336, 256)),
                                         (synth.Q8_0, (3, 2048, 512)), (synth.Q2_K, (2, 2048, 384)),
                                         (synth.IQ2_XXS, (1, 7168, 256)), (synth.MXFP4, (5, 2048, 320))])
def test_two_calls_in_a_row_match_the_allocating_entry(type_id, mkn):
    import torch

    m, k, n = mkn
    raw = synth.random_weight(type_id, n, k, seed=n)
    q = QTensor.from_bytes(type_id, raw)
    for call in range(2):
        lhs = synth.random_activations(m, k, seed=100 * call + m) * np.float32(1.0 + 3.0 * call)
        x = torch.from_numpy(lhs).cuda()
        want = torch.empty(m, n, device="cuda")
        got = torch.full((m, n), 7.25, device="cuda")
        q.matmul_t_dev(mkn, x, want)
        noalloc(q, mkn, x, got)
        torch.cuda.synchronize()
        what = f"{synth.NAMES[type_id]} {mkn} call {call}"
        assert_close(got.cpu().numpy(), want.cpu().numpy(), tol=TOL, what=what + " vs jq_matmul_t_dev")
        assert_close(got.cpu().numpy(), oracle.matmul_t(type_id, mkn, lhs, raw), tol=TOL, what=what + " vs oracle")


def test_a_call_leaves_free_device_memory_unchanged():
    """Once every kernel variant involved has run once (the first launch of a kernel may make the driver load its
    code), calls - including one whose planes would fit shared memory - neither take nor return device memory."""
    import torch

    shapes = [(synth.Q4_K, (8, 14336, 256)), (synth.Q4_K, (1, 1024, 512)), (synth.Q8_0, (4, 8192, 128))]
    qs = [(QTensor.from_bytes(t, synth.random_weight(t, mkn[2], mkn[1], seed=3)), mkn) for t, mkn in shapes]
    bufs = [(torch.randn(m, k, device="cuda"), torch.empty(m, n, device="cuda")) for _, (m, k, n) in qs]
    for (q, mkn), (x, y) in zip(qs, bufs):    # first calls: symbol address, kernel attributes, code loading
        noalloc(q, mkn, x, y)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for (q, mkn), (x, y) in zip(qs, bufs):
        noalloc(q, mkn, x, y)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before


def test_sizes_beyond_the_built_in_array_are_refused():
    import torch

    q = QTensor.from_bytes(synth.Q8_0, synth.random_weight(synth.Q8_0, 16, 262144, seed=1))
    x = torch.zeros(8, 262144, device="cuda")
    y = torch.full((8, 16), 3.5, device="cuda")
    with pytest.raises(JoshuaB200Error, match="built-in array holds") as err:
        noalloc(q, (8, 262144, 16), x, y)
    assert err.value.code == _lib.E_TOO_LARGE
    torch.cuda.synchronize()
    assert bool((y == 3.5).all())  # nothing ran
    small = QTensor.from_bytes(synth.Q4_K, synth.random_weight(synth.Q4_K, 16, 256, seed=2))
    with pytest.raises(JoshuaB200Error, match="1..8 rows") as err:
        noalloc(small, (9, 256, 16), torch.zeros(9, 256, device="cuda"), torch.zeros(9, 16, device="cuda"))
    assert err.value.code == _lib.E_TOO_LARGE
