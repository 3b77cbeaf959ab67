"""The oracle's Q8_0 / Q2_K / Q4_K kernels.

The reference tree holds no golden vectors for these types (its tests compare
against candle, which is absent here), so the bit positions are guarded by
hand-computed known answers and by a second, independently written numpy
decoder; the matmul is checked the way src/kquant_dot.rs:832-879 does it
(against a sequential product over decoded weights) on the reference's own
shapes (src/kquant_dot.rs:893-929), odd n and m included.
"""
import numpy as np
import pytest

import oracle
from joshua_b200 import synth
from tests import np_decode

F16_ONE = (0x00, 0x3C)
F16_HALF = (0x00, 0x38)
F16_TWO = (0x00, 0x40)


def test_block_sizes():
    assert oracle.block_size(oracle.Q8_0) == (32, 34)
    assert oracle.block_size(oracle.Q2_K) == (256, 84)
    assert oracle.block_size(oracle.Q4_K) == (256, 144)


def test_q8_0_known_answer():
    blk = np.zeros(34, np.uint8)
    blk[0:2] = F16_HALF
    blk[2:] = np.arange(-16, 16).astype(np.int8).view(np.uint8)
    out = oracle.dequantize(oracle.Q8_0, blk)
    assert np.array_equal(out, np.arange(-16, 16, dtype=np.float32) * 0.5)


def test_q4k_known_answer_bit_positions():
    blk = np.zeros(144, np.uint8)
    blk[0:2], blk[2:4] = F16_ONE, F16_HALF  # d = 1, dmin = 0.5
    s = blk[4:16]
    # pair 0: sc = 5, m = 2; pair 1: sc = 7, m = 0
    s[0], s[4] = 5, 2
    s[1], s[5] = 7, 0
    # pair 4: sc = 0x2A (low nibble of s[8] = 0xA, top two bits of s[0] = 2), m = 0x13
    s[0] |= 2 << 6
    s[4] |= 1 << 6
    s[8] = 0x0A | (0x3 << 4)
    q = blk[16:]
    q[0] = 0x93   # value 0 = 3 (pair 0), value 32 = 9 (pair 1)
    q[31] = 0x0F  # value 31 = 15
    q[64 + 5] = 0x0C  # value 128 + 5 = 12 (pair 4)
    out = oracle.dequantize(oracle.Q4_K, blk)
    assert out[0] == 1 * 5 * 3 - 0.5 * 2
    assert out[31] == 1 * 5 * 15 - 0.5 * 2
    assert out[32] == 1 * 7 * 9 - 0
    assert out[1] == -1.0  # q = 0 in pair 0
    assert out[128 + 5] == 1 * 0x2A * 12 - 0.5 * 0x13
    assert out[128 + 6] == -0.5 * 0x13


def test_q2k_known_answer_bit_positions():
    blk = np.zeros(84, np.uint8)
    blk[80:82], blk[82:84] = F16_TWO, F16_ONE  # d = 2, dmin = 1
    scales, qs = blk[0:16], blk[16:80]
    scales[0] = 0x35   # group 0: scale 5, min 3
    scales[3] = 0x12   # group 3 (values 48..63): scale 2, min 1
    scales[8 + 6] = 0x0F  # super-group 1, group 6 (values 128+96 .. 128+111): scale 15, min 0
    qs[0] = 0b11_10_01_11    # values 0, 32, 64, 96 = 3, 1, 2, 3
    qs[16 + 4] = 0b00_00_10_00  # byte 20: value 32 + 20 = 52 -> q = 2 (group 3)
    qs[32 + 7] = 0b01_00_00_00  # super-group 1, byte 7: value 128 + 96 + 7 -> q = 1
    out = oracle.dequantize(oracle.Q2_K, blk)
    assert out[0] == 2 * 5 * 3 - 1 * 3
    assert out[1] == -3.0
    assert out[52] == 2 * 2 * 2 - 1 * 1
    assert out[128 + 96 + 7] == 2 * 15 * 1
    assert out[32] == 0.0  # group 2 has scale 0, min 0 (q = 1 there)


@pytest.mark.parametrize("type_id", [oracle.Q8_0, oracle.Q2_K, oracle.Q4_K])
def test_numpy_restatement_agrees(type_id):
    raw = synth.random_weight(type_id, 8, 1024, seed=3)
    two_step = oracle.dequantize(type_id, raw, two_step=True)
    assert np.array_equal(two_step.view(np.uint32), np_decode.DECODERS[type_id](raw).view(np.uint32))
    fused = oracle.dequantize(type_id, raw)
    # one fused rounding vs two: at most one unit in the last place apart
    ulp = np.spacing(np.maximum(np.abs(fused), np.abs(two_step)))
    assert np.all(np.abs(fused - two_step) <= ulp)


CASES = {
    oracle.Q8_0: [(1, 256, 40), (3, 512, 17), (1, 256, 64), (5, 128, 9)],
    oracle.Q2_K: [(1, 256, 40), (3, 512, 11), (5, 768, 9)],
    oracle.Q4_K: [(1, 256, 40), (3, 512, 13), (4, 768, 25)],
}


@pytest.mark.parametrize("type_id,mkn", [(t, c) for t, cs in CASES.items() for c in cs])
def test_fused_matmul_matches_decoded_product(type_id, mkn):
    m, k, n = mkn
    raw = synth.random_weight(type_id, n, k, seed=n)
    lhs = synth.random_activations(m, k, seed=k)
    got = oracle.matmul_t(type_id, mkn, lhs, raw)
    w = oracle.dequantize(type_id, raw).reshape(n, k).astype(np.float64)
    want = lhs.astype(np.float64) @ w.T
    assert np.all(np.abs(got - want) <= 1e-3 * np.maximum(np.abs(want), 1.0))
    seq = oracle.matmul_t(type_id, mkn, lhs, raw, scalar=True, threads=1)
    assert np.all(np.abs(got - seq) <= 2e-2 * np.maximum(np.abs(seq), 1.0))


@pytest.mark.parametrize("type_id,mkn", [(oracle.Q2_K, (1, 7680, 2048)), (oracle.Q4_K, (1, 2048, 7680)),
                                         (oracle.Q8_0, (1, 4096, 4096))])
def test_model_shapes(type_id, mkn):
    m, k, n = mkn
    raw = synth.random_weight(type_id, n, k, seed=1)
    lhs = synth.random_activations(m, k, seed=2)
    got = oracle.matmul_t(type_id, mkn, lhs, raw)
    w = oracle.dequantize(type_id, raw).reshape(n, k).astype(np.float64)
    want = lhs.astype(np.float64) @ w.T
    assert np.all(np.abs(got - want) <= 1e-3 * np.maximum(np.abs(want), 1.0))


@pytest.mark.parametrize("type_id", [oracle.Q8_0, oracle.Q2_K, oracle.Q4_K])
def test_threaded_matches_serial_bit_exact(type_id):
    mkn = (3, 256, 24)
    raw = synth.random_weight(type_id, 24, 256, seed=9)
    lhs = synth.random_activations(3, 256, seed=10)
    par = oracle.matmul_t(type_id, mkn, lhs, raw, threads=0)
    ser = oracle.matmul_t(type_id, mkn, lhs, raw, threads=1)
    assert np.array_equal(par.view(np.uint32), ser.view(np.uint32))


@pytest.mark.parametrize("type_id", [oracle.Q8_0, oracle.Q2_K, oracle.Q4_K])
def test_shape_errors_and_noops(type_id):
    elems, nbytes = oracle.block_size(type_id)
    raw = synth.random_weight(type_id, 8, 256, seed=0)
    with pytest.raises(oracle.OracleError, match="not a multiple"):
        oracle.matmul_t(type_id, (1, 100, 8), np.zeros(100), raw)
    with pytest.raises(oracle.OracleError, match="blocks, expected"):
        oracle.matmul_t(type_id, (1, 256, 7), np.zeros(256), raw)
    with pytest.raises(oracle.OracleError, match="lhs/dst sized"):
        oracle.matmul_t(type_id, (2, 256, 8), np.zeros(256), raw, dst_len=16)
    with pytest.raises(oracle.OracleError, match="whole number"):
        oracle.matmul_t(type_id, (1, 256, 8), np.zeros(256), raw[:-1])
    # m == 0 or n == 0 is an accepted no-op (src/quant_matmul.rs:176-178)
    assert oracle.matmul_t(type_id, (0, 256, 8), np.zeros(0), raw).size == 0
    assert oracle.matmul_t(type_id, (2, 256, 0), np.zeros(512), raw[:0]).size == 0


def test_assigns_into_a_dirty_destination():
    raw = synth.random_weight(oracle.Q4_K, 9, 256, seed=4)
    lhs = synth.random_activations(2, 256, seed=5)
    fresh = oracle.matmul_t(oracle.Q4_K, (2, 256, 9), lhs, raw)
    dirty = np.full((2, 9), 123.75, dtype=np.float32)
    oracle.matmul_t(oracle.Q4_K, (2, 256, 9), lhs, raw, dst=dirty)
    assert np.array_equal(fresh, dirty)
