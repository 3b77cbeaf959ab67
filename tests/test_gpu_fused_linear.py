"""The quantized linear with the RMS norm in its prologue and the residual add in its epilogue against the
separate kernels (norm kernel, plain matmul, add), and the gate/up SwiGLU pair with the norm folded in."""
import numpy as np
import pytest

from joshua_b200 import synth

pytestmark = pytest.mark.gpu

TYPES = [synth.Q8_0, synth.Q2_K, synth.Q4_K, synth.IQ2_XXS, synth.MXFP4]


def _close(got, want, tol=1e-5):
    assert float((got - want).abs().max()) <= tol * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("type_id", TYPES)
@pytest.mark.parametrize("m,k,n", [(1, 1024, 272), (3, 2048, 130), (8, 4096, 64), (2, 512, 40)])
@pytest.mark.parametrize("use_norm,use_res", [(True, False), (False, True), (True, True)])
def test_linear_with_norm_and_residual(type_id, m, k, n, use_norm, use_res):
    import torch

    from joshua_b200 import _lib
    from joshua_b200.qtensor import QTensor

    L = _lib.lib()
    w = QTensor.from_bytes(type_id, synth.random_weight(type_id, n, k, 3))
    g = torch.Generator(device="cuda").manual_seed(m * 1000 + n)
    x = torch.randn(m, k, device="cuda", generator=g)
    nw = 1.0 + 0.1 * torch.randn(k, device="cuda", generator=g)
    res = torch.randn(m, n, device="cuda", generator=g)
    s = torch.cuda.current_stream().cuda_stream
    xn = torch.empty_like(x)
    if use_norm:
        _lib.check(L.jq_rmsnorm_dev(x.data_ptr(), None, nw.data_ptr(), 1e-5, m, k, None, xn.data_ptr(), s))
    else:
        xn.copy_(x)
    want = torch.empty(m, n, device="cuda")
    _lib.check(L.jq_matmul_t_dev(w._h, m, k, n, xn.data_ptr(), want.data_ptr(), s))
    if use_res:
        want += res
    got = res.clone() if use_res else torch.empty(m, n, device="cuda")   # residual in place
    _lib.check(L.jq_matmul_norm_dev(w._h, m, k, n, x.data_ptr(), nw.data_ptr() if use_norm else None, 1e-5,
                                    got.data_ptr() if use_res else None, got.data_ptr(), s))
    torch.cuda.synchronize()
    _close(got, want)


@pytest.mark.parametrize("type_id", [synth.Q4_K, synth.Q8_0])
@pytest.mark.parametrize("m", [1, 4])
def test_swiglu_pair_with_norm(type_id, m):
    import torch

    from joshua_b200 import _lib
    from joshua_b200.qtensor import QTensor

    L = _lib.lib()
    k, n = 1024, 304
    gate = QTensor.from_bytes(type_id, synth.random_weight(type_id, n, k, 1))
    up = QTensor.from_bytes(type_id, synth.random_weight(type_id, n, k, 2))
    g = torch.Generator(device="cuda").manual_seed(m)
    x = torch.randn(m, k, device="cuda", generator=g) * 0.05
    nw = 1.0 + 0.1 * torch.randn(k, device="cuda", generator=g)
    s = torch.cuda.current_stream().cuda_stream
    xn = torch.empty_like(x)
    _lib.check(L.jq_rmsnorm_dev(x.data_ptr(), None, nw.data_ptr(), 1e-6, m, k, None, xn.data_ptr(), s))
    want = torch.empty(m, n, device="cuda")
    _lib.check(L.jq_matmul_swiglu_dev(gate._h, up._h, m, k, n, xn.data_ptr(), want.data_ptr(), 0.0, s))
    got = torch.empty(m, n, device="cuda")
    _lib.check(L.jq_matmul_swiglu_norm_dev(gate._h, up._h, m, k, n, x.data_ptr(), nw.data_ptr(), 1e-6, got.data_ptr(),
                                           0.0, s))
    torch.cuda.synchronize()
    _close(got, want, 1e-4)
