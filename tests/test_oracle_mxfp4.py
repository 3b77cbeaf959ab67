"""The oracle's MXFP4 decode and matmul against the reference's known answers.

Restates the unit tests of src/mxfp4.rs:281-458 (every expected value below is
the one asserted there).
"""
import numpy as np
import pytest

import oracle
from tests import np_decode


def block(e, qs):
    return np.array([e] + list(qs), dtype=np.uint8)


def spread_rhs(n, blocks_per_row):
    """The deterministic code spread of src/mxfp4.rs:356-369."""
    out = []
    for r in range(n):
        for b in range(blocks_per_row):
            qs = [((j + r * 3 + b * 5) % 16) | (((j + r) % 16) << 4) for j in range(16)]
            out.append(block(127 + (r % 3), qs))
    return np.concatenate(out)


def test_e8m0_decodes_to_powers_of_two():
    assert oracle.e8m0_to_f32(127) == 1.0
    assert oracle.e8m0_to_f32(128) == 2.0
    assert oracle.e8m0_to_f32(126) == 0.5
    assert oracle.e8m0_to_f32(130) == 8.0
    tiny = oracle.e8m0_to_f32(0)
    assert tiny > 0 and tiny.view(np.uint32) == 0x00400000
    assert oracle.e8m0_to_f32(0xFF) is None


def test_block_uses_split_half_nibble_order():
    out = oracle.dequantize(oracle.MXFP4, block(127, [0x17] + [0] * 15))
    assert out[0] == 6.0 and out[16] == 0.5 and out[1] == 0.0


def test_scale_multiplies_every_element():
    qs = [0] * 16
    qs[3] = 0x0F
    assert oracle.dequantize(oracle.MXFP4, block(129, qs))[3] == -24.0


def test_nan_scale_decodes_to_zeros():
    out = oracle.dequantize(oracle.MXFP4, block(0xFF, [0xFF] * 16))
    assert np.all(out == 0.0)


def test_full_e2m1_table():
    out = oracle.dequantize(oracle.MXFP4, block(127, range(16)))
    assert np.array_equal(out[:16], np_decode.E2M1)
    assert oracle.block_size(oracle.MXFP4) == (32, 17)


def test_numpy_restatement_agrees_bit_for_bit():
    rng = np.random.default_rng(5)
    raw = rng.integers(0, 256, size=(64, 17), dtype=np.uint8)
    raw[:4, 0] = [0, 1, 254, 255]
    a = oracle.dequantize(oracle.MXFP4, raw.reshape(-1))
    b = np_decode.mxfp4(raw.reshape(-1))
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_matmul_matches_explicit_dequantized_reference():
    m, k, n = 2, 64, 3
    rhs = spread_rhs(n, k // 32)
    lhs = (np.arange(m * k, dtype=np.float32) % 7.0 - 3.0).reshape(m, k)
    got = oracle.matmul_t(oracle.MXFP4, (m, k, n), lhs, rhs)
    w = oracle.dequantize(oracle.MXFP4, rhs).reshape(n, k)
    want = lhs.astype(np.float64) @ w.astype(np.float64).T
    assert np.all(np.abs(got - want) < 1e-3)


def test_matmul_assigns_rather_than_accumulating():
    m, k, n = 1, 32, 2
    rhs = np.concatenate([block(127, [0x21] * 16), block(128, [0x34] * 16)])
    lhs = (np.arange(k) % 5).astype(np.float32) - 2.0
    fresh = oracle.matmul_t(oracle.MXFP4, (m, k, n), lhs, rhs)
    dirty = np.full((m, n), 123.75, dtype=np.float32)
    oracle.matmul_t(oracle.MXFP4, (m, k, n), lhs, rhs, dst=dirty)
    assert np.array_equal(fresh, dirty)


def test_threaded_matches_serial_bit_exact():
    m, k, n = 4, 1024, 23
    rhs = spread_rhs(n, k // 32)
    i = np.arange(m * k, dtype=np.int64)
    lhs = (((i * 104729) % 1000).astype(np.float32) / np.float32(100.0) - np.float32(5.0)).reshape(m, k)
    par = oracle.matmul_t(oracle.MXFP4, (m, k, n), lhs, rhs, threads=0)
    ser = oracle.matmul_t(oracle.MXFP4, (m, k, n), lhs, rhs, threads=1)
    assert np.array_equal(par.view(np.uint32), ser.view(np.uint32))


def test_partial_block_is_rejected():
    oracle.dequantize(oracle.MXFP4, np.zeros(17, np.uint8))
    oracle.dequantize(oracle.MXFP4, np.zeros(34, np.uint8))
    with pytest.raises(oracle.OracleError, match="whole number"):
        oracle.dequantize(oracle.MXFP4, np.zeros(20, np.uint8))
    with pytest.raises(oracle.OracleError, match="not a multiple"):
        oracle.matmul_t(oracle.MXFP4, (1, 40, 1), np.zeros(40), np.zeros(17, np.uint8))
