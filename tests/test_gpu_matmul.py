"""matmul_t through the C ABI against the oracle: the reference's own shapes and error cases."""
import numpy as np
import pytest

import oracle
from joshua_b200 import synth
from joshua_b200.qtensor import QTensor, QMatMul
from joshua_b200._lib import JoshuaB200Error
from tests.gpu_util import assert_close, bits
from tests.test_oracle_iq2xxs import fixture_rhs, lhs_pattern
from tests.test_oracle_mxfp4 import spread_rhs

pytestmark = pytest.mark.gpu

# (m, k, n) of the reference's unit tests (src/kquant_dot.rs:893-929, src/quant_matmul.rs:498-533,
# src/iq2xxs.rs:761-873, src/mxfp4.rs:354-423): odd n, m off the 4-row tile.
SMALL = {
    synth.Q8_0: [(1, 256, 40), (3, 512, 17), (1, 256, 64), (5, 128, 9), (3, 256, 24), (2, 256, 8)],
    synth.Q2_K: [(1, 256, 40), (3, 512, 11), (5, 768, 9), (3, 256, 24), (2, 256, 8)],
    synth.Q4_K: [(1, 256, 40), (3, 512, 13), (4, 768, 25), (3, 256, 24), (2, 256, 8)],
    synth.IQ2_XXS: [(3, 512, 7), (3, 1024, 11), (4, 1024, 23)],
    synth.MXFP4: [(2, 64, 3), (1, 32, 2), (4, 1024, 23), (2, 64, 6)],
}
# decode shapes of the benchmark configurations, and batches up to and past the 8-row tile
MODEL = [
    (synth.Q4_K, (1, 4096, 4096)), (synth.Q8_0, (1, 4096, 4096)), (synth.Q2_K, (1, 4096, 4096)),
    (synth.Q2_K, (1, 7680, 2048)), (synth.Q4_K, (1, 2048, 7680)), (synth.Q8_0, (32, 4096, 4096)),
    (synth.Q4_K, (8, 4096, 1024)), (synth.Q4_K, (1, 14336, 512)), (synth.Q4_K, (7, 2048, 768)),
    (synth.Q4_K, (13, 768, 2048)), (synth.IQ2_XXS, (1, 7168, 2048)), (synth.IQ2_XXS, (5, 2048, 7168)),
    (synth.MXFP4, (1, 7168, 2048)), (synth.MXFP4, (16, 2048, 7168)), (synth.Q8_0, (2, 7168, 1536)),
]


@pytest.mark.parametrize("type_id,mkn", [(t, c) for t, cs in SMALL.items() for c in cs] + MODEL)
def test_matmul_matches_oracle(type_id, mkn):
    m, k, n = mkn
    raw = synth.random_weight(type_id, n, k, seed=n + k)
    lhs = synth.random_activations(m, k, seed=m)
    got = QTensor.from_bytes(type_id, raw).matmul_t(mkn, lhs)
    want = oracle.matmul_t(type_id, mkn, lhs, raw)
    assert_close(got, want, what=f"{synth.NAMES[type_id]} {mkn}")


@pytest.mark.parametrize("type_id", synth.GENERIC_TYPES)
@pytest.mark.parametrize("mkn", [(1, 256, 40), (3, 512, 13), (8, 1024, 64), (40, 512, 24), (1, 4096, 256)])
def test_generic_path_types_match_oracle(type_id, mkn):
    """The block types the reference serves by decoding a row and dotting it (src/quant_matmul.rs:228-249): here
    the exact-decode float kernel, any batch."""
    m, k, n = mkn
    raw = synth.random_weight(type_id, n, k, seed=n + k)
    lhs = synth.random_activations(m, k, seed=m)
    q = QTensor.from_bytes(type_id, raw)
    got = q.matmul_t(mkn, lhs)
    assert_close(got, oracle.matmul_t(type_id, mkn, lhs, raw), what=f"{synth.NAMES[type_id]} {mkn}")
    assert np.array_equal(bits(got), bits(q.matmul_t(mkn, lhs)))      # run-to-run bit equality


def test_iq2xxs_golden_block_fixture():
    for mkn, mult in [((3, 512, 7), 7919), ((3, 1024, 11), 7919), ((4, 1024, 23), 104729)]:
        m, k, n = mkn
        rhs, lhs = fixture_rhs(k, n), lhs_pattern(m, k, mult)
        got = QTensor.from_bytes(synth.IQ2_XXS, rhs).matmul_t(mkn, lhs)
        assert_close(got, oracle.matmul_t(synth.IQ2_XXS, mkn, lhs, rhs), tol=1e-4)


def test_mxfp4_reference_fixtures():
    m, k, n = 2, 64, 3
    rhs = spread_rhs(n, k // 32)
    lhs = (np.arange(m * k, dtype=np.float32) % 7.0 - 3.0).reshape(m, k)
    got = QTensor.from_bytes(synth.MXFP4, rhs).matmul_t((m, k, n), lhs)
    assert np.all(np.abs(got - oracle.matmul_t(synth.MXFP4, (m, k, n), lhs, rhs)) < 1e-3)
    # a per-expert slice of a borrowed tensor (src/mmap_tensor.rs:923-954): rows 3..6 of a 6-row tensor
    full = spread_rhs(6, 2)
    q = QTensor.from_bytes(synth.MXFP4, full)
    part = q.slice_blocks(3 * 2, 3 * 2)
    got = part.matmul_t((m, k, 3), lhs)
    want = oracle.matmul_t(synth.MXFP4, (m, k, 3), lhs, full[3 * 2 * 17:])
    assert np.all(np.abs(got - want) < 1e-3)


@pytest.mark.parametrize("type_id", list(SMALL))
def test_assigns_into_dirty_destination_and_is_deterministic(type_id):
    elems, _ = synth.BLOCK[type_id]
    m, k, n = 3, 4 * elems if elems == 256 else 256, 19
    raw = synth.random_weight(type_id, n, k, seed=2)
    lhs = synth.random_activations(m, k, seed=3)
    q = QTensor.from_bytes(type_id, raw)
    fresh = q.matmul_t((m, k, n), lhs)
    dirty = np.full((m, n), 123.75, dtype=np.float32)
    q.matmul_t((m, k, n), lhs, dst=dirty)
    assert np.array_equal(bits(fresh), bits(dirty))
    assert np.array_equal(bits(fresh), bits(q.matmul_t((m, k, n), lhs)))


@pytest.mark.parametrize("type_id", list(SMALL))
def test_shape_errors_and_noops(type_id):
    elems, nbytes = synth.BLOCK[type_id]
    k = 256
    raw = synth.random_weight(type_id, 8, k, seed=0)
    q = QTensor.from_bytes(type_id, raw)
    with pytest.raises(JoshuaB200Error, match="not a multiple"):
        q.matmul_t((1, 100, 8), np.zeros(100, np.float32))
    with pytest.raises(JoshuaB200Error, match="blocks, expected"):
        q.matmul_t((1, k, 7), np.zeros(k, np.float32))
    with pytest.raises(JoshuaB200Error, match="lhs/dst sized"):
        q.matmul_t((2, k, 8), np.zeros(k, np.float32), dst_len=16)
    with pytest.raises(JoshuaB200Error, match="lhs/dst sized"):
        q.matmul_t((1, k, 8), np.zeros(k, np.float32), dst_len=7)
    assert q.matmul_t((0, k, 8), np.zeros(0, np.float32)).size == 0
    empty = QTensor.from_bytes(type_id, raw[:0])
    assert empty.matmul_t((2, k, 0), np.zeros(2 * k, np.float32)).size == 0


@pytest.mark.parametrize("type_id", [synth.IQ2_XXS, synth.MXFP4, synth.Q4_K])
def test_f16_entry(type_id):
    m, k, n = 3, 512, 21
    raw = synth.random_weight(type_id, n, k, seed=7)
    lhs16 = synth.random_activations(m, k, seed=8).astype(np.float16)
    got = QTensor.from_bytes(type_id, raw).matmul_t_f16((m, k, n), lhs16)
    want = oracle.matmul_t(type_id, (m, k, n), lhs16.astype(np.float32), raw).astype(np.float16)
    assert_close(got.astype(np.float32), want.astype(np.float32), tol=2e-3)


def test_qmatmul_forward_on_device_tensors():
    import torch

    n, k = 96, 512
    raw = synth.random_weight(synth.Q4_K, n, k, seed=4)
    mm = QMatMul.from_qtensor(QTensor.from_bytes(synth.Q4_K, raw), (n, k))
    x = torch.randn(2, 3, k, device="cuda")
    y = mm.forward(x)
    assert y.shape == (2, 3, n)
    want = oracle.matmul_t(synth.Q4_K, (6, k, n), x.reshape(6, k).cpu().numpy(), raw)
    assert_close(y.reshape(6, n).cpu().numpy(), want)
    with pytest.raises(JoshuaB200Error):
        QMatMul.from_qtensor(QTensor.from_bytes(synth.Q4_K, raw), (n + 1, k))
