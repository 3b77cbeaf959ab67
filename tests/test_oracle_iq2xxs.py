"""The oracle's IQ2_XXS decode and matmul against the reference's golden vectors.

Restates the unit tests of src/iq2xxs.rs:712-903.  The golden data
(`golden/iq2xxs_blocks.bin`, 4 blocks; `golden/iq2xxs_ref.txt`, 1024 values)
are the reference's tests/data files: values produced by llama.cpp's own
`dequantize_row_iq2_xxs`.
"""
import numpy as np
import pytest

import oracle
from tests import np_decode

GOLDEN = np_decode.GOLDEN
BLOCKS = np.frombuffer((GOLDEN / "iq2xxs_blocks.bin").read_bytes(), dtype=np.uint8)
WANT = np.array([float(x) for x in (GOLDEN / "iq2xxs_ref.txt").read_text().split()], dtype=np.float32)


def fixture_rhs(k, n):
    """n rows of k columns built by cycling the 4 golden blocks (src/iq2xxs.rs:819-831)."""
    blocks = BLOCKS.reshape(4, 66)
    idx = np.arange(n * (k // 256)) % 4
    return blocks[idx].reshape(-1)


def lhs_pattern(m, k, mult=7919):
    i = np.arange(m * k, dtype=np.int64)
    return (((i * mult) % 1000).astype(np.float32) / np.float32(100.0) - np.float32(5.0)).reshape(m, k)


def test_dequant_matches_llamacpp_golden_vectors():
    got = oracle.dequantize(oracle.IQ2_XXS, BLOCKS)
    assert got.shape == WANT.shape == (1024,)
    assert np.all(np.abs(got - WANT) <= 1e-6 * np.maximum(np.abs(WANT), 1.0))


def test_numpy_restatement_matches_golden_and_oracle_bit_for_bit():
    got = np_decode.iq2xxs(BLOCKS)
    assert np.all(np.abs(got - WANT) <= 1e-6 * np.maximum(np.abs(WANT), 1.0))
    assert np.array_equal(got.view(np.uint32), oracle.dequantize(oracle.IQ2_XXS, BLOCKS).view(np.uint32))


def test_block_layout_is_66_bytes():
    assert oracle.block_size(oracle.IQ2_XXS) == (256, 66)
    blk = np.zeros(66, dtype=np.uint8)
    blk[1] = 0x3C  # d = 1.0
    assert np.all(np.isfinite(oracle.dequantize(oracle.IQ2_XXS, blk)))


def test_dequant_is_bounded():
    blk = np.full(66, 0xFF, dtype=np.uint8)
    blk[0], blk[1] = 0, 0x3C
    out = oracle.dequantize(oracle.IQ2_XXS, blk)
    assert np.all(np.abs(out) <= 43.0 * 0.25 * 15.5 + 1e-6)


@pytest.mark.parametrize("mkn", [(3, 512, 7), (3, 1024, 11), (4, 1024, 23)])
def test_matmul_matches_naive_f32(mkn):
    m, k, n = mkn
    rhs = fixture_rhs(k, n)
    lhs = lhs_pattern(m, k)
    got = oracle.matmul_t(oracle.IQ2_XXS, mkn, lhs, rhs)
    w = oracle.dequantize(oracle.IQ2_XXS, rhs).reshape(n, k)
    want = np.zeros((m, n), dtype=np.float32)
    for i in range(m):
        for j in range(n):
            acc = np.float32(0)
            for v in lhs[i] * w[j]:
                acc = np.float32(acc + v)
            want[i, j] = acc
    assert np.all(np.abs(got - want) <= 1e-4 * np.maximum(np.abs(want), 1.0))


def test_avx2_and_scalar_paths_agree():
    mkn = (3, 1024, 11)
    rhs, lhs = fixture_rhs(1024, 11), lhs_pattern(3, 1024)
    fast = oracle.matmul_t(oracle.IQ2_XXS, mkn, lhs, rhs)
    scalar = oracle.matmul_t(oracle.IQ2_XXS, mkn, lhs, rhs, scalar=True, threads=1)
    assert np.all(np.abs(fast - scalar) <= 1e-4 * np.maximum(np.abs(scalar), 1.0))


def test_threaded_matches_serial_bit_exact():
    mkn = (4, 1024, 23)
    rhs, lhs = fixture_rhs(1024, 23), lhs_pattern(4, 1024, 104729)
    par = oracle.matmul_t(oracle.IQ2_XXS, mkn, lhs, rhs, threads=0)
    ser = oracle.matmul_t(oracle.IQ2_XXS, mkn, lhs, rhs, threads=1)
    assert np.array_equal(par.view(np.uint32), ser.view(np.uint32))


def test_matmul_rejects_bad_shapes():
    with pytest.raises(oracle.OracleError, match="not a multiple"):
        oracle.matmul_t(oracle.IQ2_XXS, (1, 100, 1), np.zeros(100), BLOCKS)
    with pytest.raises(oracle.OracleError, match="blocks, expected"):
        oracle.matmul_t(oracle.IQ2_XXS, (1, 256, 1), np.zeros(256), BLOCKS)
    with pytest.raises(oracle.OracleError, match="lhs/dst sized"):
        oracle.matmul_t(oracle.IQ2_XXS, (2, 256, 4), np.zeros(256), BLOCKS, dst_len=8)
    with pytest.raises(oracle.OracleError, match="whole number"):
        oracle.dequantize(oracle.IQ2_XXS, BLOCKS[:100])
