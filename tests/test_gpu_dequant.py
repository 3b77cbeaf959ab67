"""Block decode on the GPU is bit-exact against the oracle (and the golden vectors)."""
import numpy as np
import pytest

import oracle
from joshua_b200 import synth
from joshua_b200.qtensor import QTensor
from joshua_b200._lib import JoshuaB200Error
from tests import np_decode
from tests.gpu_util import bits

pytestmark = pytest.mark.gpu
TYPES = [synth.Q8_0, synth.Q2_K, synth.Q4_K, synth.IQ2_XXS, synth.MXFP4]


@pytest.mark.parametrize("type_id", TYPES)
@pytest.mark.parametrize("two_step", [False, True])
def test_dequant_bit_exact(type_id, two_step):
    elems, nbytes = synth.BLOCK[type_id]
    raw = synth.random_blocks(type_id, 4099, np.random.default_rng(type_id)).reshape(-1)
    q = QTensor.from_bytes(type_id, raw)
    got = q.dequantize(4099 * elems, two_step=two_step)
    want = oracle.dequantize(type_id, raw, two_step=two_step)
    assert np.array_equal(bits(got), bits(want))


@pytest.mark.parametrize("type_id", synth.GENERIC_TYPES)
def test_generic_path_types_dequant_bit_exact(type_id):
    """Q4_0 .. Q8_K (the reference's `decode_raw_to_f32` ids 2, 3, 6, 7, 9, 11, 13, 14, 15, src/quant_matmul.rs:86-100)
    against the oracle's scalar decoders, including the embedding gather."""
    elems, nbytes = synth.BLOCK[type_id]
    raw = synth.random_blocks(type_id, 1031, np.random.default_rng(type_id)).reshape(-1)
    q = QTensor.from_bytes(type_id, raw)
    want = oracle.dequantize(type_id, raw)
    assert np.array_equal(bits(q.dequantize(1031 * elems)), bits(want))
    hidden = 2 * max(elems, 128)
    rows = 1031 * elems // hidden
    raw = raw[: rows * (hidden // elems) * nbytes]
    ids = np.array([rows - 1, 0, 5, 5], dtype=np.uint32)
    got = QTensor.from_bytes(type_id, raw).embedding(ids, rows, hidden)
    assert np.array_equal(bits(got), bits(want[: rows * hidden].reshape(rows, hidden)[ids]))


def test_iq2xxs_golden_vectors():
    raw = (np_decode.GOLDEN / "iq2xxs_blocks.bin").read_bytes()
    want = np.array([float(x) for x in (np_decode.GOLDEN / "iq2xxs_ref.txt").read_text().split()], dtype=np.float32)
    got = QTensor.from_bytes(synth.IQ2_XXS, raw).dequantize(1024)
    assert np.all(np.abs(got - want) <= 1e-6 * np.maximum(np.abs(want), 1.0))


def test_mxfp4_known_answers_and_special_scales():
    def block(e, qs):
        return np.array([e] + list(qs), dtype=np.uint8)

    raw = np.concatenate([
        block(127, [0x17] + [0] * 15),     # split-half order: out[0] = 6, out[16] = 0.5
        block(129, [0, 0, 0, 0x0F] + [0] * 12),  # -6 * 4
        block(0xFF, [0xFF] * 16),          # reserved scale -> zeros
        block(0, range(16)),               # 2^-127 denormal scale
        block(127, range(16)),             # the E2M1 table
        block(254, [0x77] * 16),           # largest finite scale
    ])
    got = QTensor.from_bytes(synth.MXFP4, raw).dequantize(6 * 32)
    assert got[0] == 6.0 and got[16] == 0.5 and got[1] == 0.0
    assert got[32 + 3] == -24.0
    assert np.all(got[64:96] == 0.0)
    assert np.array_equal(got[128:144], np_decode.E2M1)
    assert np.array_equal(bits(got), bits(oracle.dequantize(synth.MXFP4, raw)))


def test_q8_0_minus_128_and_extreme_scales():
    raw = synth.random_blocks(synth.Q8_0, 8, np.random.default_rng(0))
    raw[0, 2:] = 0x80
    raw[1, 0:2] = (0xFF, 0x7B)  # 65504
    raw[2, 0:2] = (0x01, 0x00)  # smallest subnormal
    raw[3, 0:2] = (0x00, 0x80)  # -0
    got = QTensor.from_bytes(synth.Q8_0, raw.reshape(-1)).dequantize(8 * 32)
    assert np.array_equal(bits(got), bits(oracle.dequantize(synth.Q8_0, raw.reshape(-1))))


@pytest.mark.parametrize("type_id", TYPES)
def test_embedding_rows(type_id):
    elems, _ = synth.BLOCK[type_id]
    rows, hidden = 37, 512
    raw = synth.random_weight(type_id, rows, hidden, seed=5)
    q = QTensor.from_bytes(type_id, raw)
    ids = np.array([0, 36, 5, 5, 17], dtype=np.uint32)
    got = q.embedding(ids, rows, hidden)
    want = oracle.dequantize(type_id, raw, two_step=True).reshape(rows, hidden)[ids]
    assert np.array_equal(bits(got), bits(want))
    with pytest.raises(JoshuaB200Error, match="out of range"):
        q.embedding(np.array([37], dtype=np.uint32), rows, hidden)
    with pytest.raises(JoshuaB200Error, match="not divisible"):
        q.embedding(ids, rows, hidden + 8)
    with pytest.raises(JoshuaB200Error, match="blocks, expected"):
        q.embedding(ids, rows + 1, hidden)


def test_size_errors():
    raw = synth.random_weight(synth.Q4_K, 2, 256, seed=1)
    with pytest.raises(JoshuaB200Error, match="whole number"):
        QTensor.from_bytes(synth.Q4_K, raw[:-1])
    with pytest.raises(JoshuaB200Error, match="unsupported"):
        QTensor.from_bytes(17, raw)      # IQ2_XS: no decoder here
    q = QTensor.from_bytes(synth.Q4_K, raw)
    with pytest.raises(JoshuaB200Error, match="output holds"):
        q.dequantize(256)
    assert q.dtype() == synth.Q4_K and q.block_size() == 256 and q.storage_size_in_bytes() == 288
    with pytest.raises(JoshuaB200Error, match="read-only"):
        q.from_float(np.zeros(512, np.float32))
    assert QTensor.from_bytes(synth.Q4_K, raw[:0]).dequantize(0).size == 0
