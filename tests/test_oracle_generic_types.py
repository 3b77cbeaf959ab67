"""The block types of the reference's generic path (Q4_0, Q4_1, Q5_0, Q5_1, Q8_1, Q3_K, Q5_K, Q6_K, Q8_K;
src/quant_matmul.rs:86-100,228-249): the C++ oracle's scalar decoders against the independently written numpy
decoders of `joshua_b200.ggml_decode`, hand-computed known answers for the bit fields, and the dequantise-row +
8-lane dot product against a float64 product.  The reference decodes these types with candle's `to_float` (not
in its tree) and holds no vectors for them: parity unpinned, anchored on the published ggml layouts."""
import numpy as np
import pytest

import oracle
from joshua_b200 import ggml_decode, synth


@pytest.mark.parametrize("type_id", synth.GENERIC_TYPES)
def test_oracle_and_numpy_decoders_agree_bit_for_bit(type_id):
    raw = synth.random_weight(type_id, 37, 4 * synth.BLOCK[type_id][0], seed=type_id)
    a = oracle.dequantize(type_id, raw)
    b = ggml_decode.dequantize(type_id, raw)
    assert a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))
    assert np.isfinite(a).all()


def f16(v):
    return np.frombuffer(np.float16(v).tobytes(), dtype=np.uint8)


def test_known_answers_q4_0_q4_1_q5_0_q5_1():
    b = np.zeros(18, np.uint8)
    b[0:2] = f16(0.5)
    b[2] = 0x1F                     # value 0 = 15 - 8 = 7, value 16 = 1 - 8 = -7
    out = oracle.dequantize(synth.Q4_0, b)
    assert out[0] == 3.5 and out[16] == -3.5 and out[1] == -4.0
    b = np.zeros(20, np.uint8)
    b[0:2], b[2:4] = f16(0.25), f16(1.0)
    b[4 + 3] = 0xA2                 # value 3 = 2, value 19 = 10
    out = oracle.dequantize(synth.Q4_1, b)
    assert out[3] == 1.5 and out[19] == 3.5 and out[0] == 1.0
    b = np.zeros(22, np.uint8)
    b[0:2] = f16(1.0)
    b[2:6] = np.frombuffer(np.uint32((1 << 5) | (1 << 21)).tobytes(), np.uint8)   # fifth bit of values 5 and 21
    b[6 + 5] = 0x93                 # value 5: 3 | 16 = 19 - 16 = 3; value 21: 9 | 16 = 25 - 16 = 9
    out = oracle.dequantize(synth.Q5_0, b)
    assert out[5] == 3.0 and out[21] == 9.0 and out[0] == -16.0
    b = np.zeros(24, np.uint8)
    b[0:2], b[2:4] = f16(2.0), f16(-1.0)
    b[4:8] = np.frombuffer(np.uint32(1 << 31).tobytes(), np.uint8)
    b[8 + 15] = 0xF0                # value 31: 15 | 16 = 31 -> 61
    out = oracle.dequantize(synth.Q5_1, b)
    assert out[31] == 61.0 and out[15] == -1.0


def test_known_answers_q6_k_q5_k_q3_k_q8():
    b = np.zeros(210, np.uint8)
    b[208:210] = f16(0.5)
    b[192:208] = 2                  # every scale 2
    b[0] = 0x07                     # ql[0]: low nibble 7 -> value 0, high nibble 0 -> value 64
    b[128] = 0b11_10_01_10          # qh[0]: values 0 / 32 / 64 / 96 get high bits 2 / 1 / 2 / 3
    out = oracle.dequantize(synth.Q6_K, b)
    assert out[0] == 0.5 * 2 * ((7 | (2 << 4)) - 32)      # 39 - 32 = 7
    assert out[32] == 0.5 * 2 * ((0 | (1 << 4)) - 32) and out[64] == 0.5 * 2 * (32 - 32) and out[96] == 0.5 * 2 * (48 - 32)
    assert out[1] == -32.0
    b = np.zeros(176, np.uint8)
    b[0:2], b[2:4] = f16(1.0), f16(0.5)
    b[4], b[8] = 3, 2               # group 0: scale 3, minimum 2
    b[16] = 0b01                    # qh[0]: fifth bit for group 0
    b[48] = 0x04                    # ql[0]: low nibble 4
    out = oracle.dequantize(synth.Q5_K, b)
    assert out[0] == 3.0 * 20 - 1.0 and out[1] == -1.0
    b = np.zeros(110, np.uint8)
    b[108:110] = f16(1.0)
    b[96] = 0x05                    # scale 0 low nibble 5, high bits 0 -> 5 - 32 = -27
    b[32] = 0b10                    # qs[0]: value 0 has low bits 2
    b[0] = 0b1                      # hmask[0] bit 0 set for value 0: nothing subtracted
    out = oracle.dequantize(synth.Q3_K, b)
    assert out[0] == -27.0 * 2 and out[1] == -27.0 * (0 - 4)
    b = np.zeros(36, np.uint8)
    b[0:2] = f16(0.5)
    b[4] = 0x80                     # -128
    assert oracle.dequantize(synth.Q8_1, b)[0] == -64.0
    b = np.zeros(292, np.uint8)
    b[0:4] = np.frombuffer(np.float32(0.125).tobytes(), np.uint8)
    b[4 + 255] = 0x7F
    assert oracle.dequantize(synth.Q8_K, b)[255] == 127 * 0.125


@pytest.mark.parametrize("type_id", synth.GENERIC_TYPES)
@pytest.mark.parametrize("mkn", [(1, 256, 40), (3, 512, 13), (5, 768, 9)])
def test_generic_matmul_matches_a_float64_product(type_id, mkn):
    m, k, n = mkn
    raw = synth.random_weight(type_id, n, k, seed=n + type_id)
    lhs = synth.random_activations(m, k, seed=m)
    got = oracle.matmul_t(type_id, mkn, lhs, raw)
    w = ggml_decode.dequantize(type_id, raw).reshape(n, k).astype(np.float64)
    want = lhs.astype(np.float64) @ w.T
    assert np.abs(got - want).max() <= 1e-4 * max(1.0, np.abs(want).max())
    serial = oracle.matmul_t(type_id, mkn, lhs, raw, threads=1)
    assert np.array_equal(got.view(np.uint32), serial.view(np.uint32))     # thread count does not change a bit
