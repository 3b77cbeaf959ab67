"""The tensor-core tile GEMM (m > 8: prefill and batched decode) against the oracle."""
import numpy as np
import pytest

import oracle
from joshua_b200 import synth
from joshua_b200.qtensor import QTensor
from tests.gpu_util import assert_close, bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tc_ctx():
    """A context that sends every batch above 8 to the tile GEMM (by default batches up to 64 run as 8-row
    slices of the decode kernel)."""
    import os

    from joshua_b200.qtensor import Context

    old = os.environ.get("JQ_SLICED_MAX_M")
    os.environ["JQ_SLICED_MAX_M"] = "0"
    try:
        ctx = Context(0)
    finally:
        if old is None:
            del os.environ["JQ_SLICED_MAX_M"]
        else:
            os.environ["JQ_SLICED_MAX_M"] = old
    return ctx

CASES = [
    (synth.Q4_K, (9, 256, 16)), (synth.Q4_K, (16, 512, 128)), (synth.Q4_K, (33, 768, 130)),
    (synth.Q4_K, (64, 4096, 256)), (synth.Q4_K, (100, 2048, 768)), (synth.Q4_K, (512, 4096, 384)),
    (synth.Q4_K, (300, 1024, 77)), (synth.Q8_0, (32, 4096, 512)), (synth.Q8_0, (129, 512, 200)),
    (synth.Q2_K, (40, 1024, 129)), (synth.Q2_K, (256, 7680, 128)), (synth.IQ2_XXS, (17, 1024, 23)),
    (synth.IQ2_XXS, (128, 7168, 256)), (synth.MXFP4, (16, 2048, 300)), (synth.MXFP4, (257, 7168, 128)),
    (synth.MXFP4, (12, 96, 40)),
]


@pytest.mark.parametrize("type_id,mkn", CASES)
def test_matches_oracle(type_id, mkn, tc_ctx):
    m, k, n = mkn
    raw = synth.random_weight(type_id, n, k, seed=n + k)
    lhs = synth.random_activations(m, k, seed=m)
    q = QTensor.from_bytes(type_id, raw, tc_ctx)
    got = q.matmul_t(mkn, lhs)
    want = oracle.matmul_t(type_id, mkn, lhs, raw)
    assert_close(got, want, what=f"{synth.NAMES[type_id]} {mkn}")
    assert np.array_equal(bits(got), bits(q.matmul_t(mkn, lhs)))  # run-to-run identical


def test_assigns_and_leaves_neighbours_alone(tc_ctx):
    m, k, n = 20, 512, 70
    raw = synth.random_weight(synth.Q4_K, n, k, seed=1)
    lhs = synth.random_activations(m, k, seed=2)
    q = QTensor.from_bytes(synth.Q4_K, raw, tc_ctx)
    dirty = np.full((m, n), 123.75, dtype=np.float32)
    q.matmul_t((m, k, n), lhs, dst=dirty)
    assert_close(dirty, oracle.matmul_t(synth.Q4_K, (m, k, n), lhs, raw))


@pytest.mark.parametrize("type_id,mkn", [(synth.Q4_K, (9, 256, 16)), (synth.Q4_K, (20, 4096, 130)), (synth.Q8_0, (64, 2048, 96)),
                                         (synth.MXFP4, (33, 1024, 40)), (synth.IQ2_XXS, (17, 1024, 23)), (synth.Q2_K, (40, 1024, 129))])
def test_sliced_batches_match_oracle(type_id, mkn):
    """Batches 9..64 through the default context: 8-row slices of the decode kernel."""
    m, k, n = mkn
    raw = synth.random_weight(type_id, n, k, seed=n + k)
    lhs = synth.random_activations(m, k, seed=m)
    q = QTensor.from_bytes(type_id, raw)
    got = q.matmul_t(mkn, lhs)
    assert_close(got, oracle.matmul_t(type_id, mkn, lhs, raw), what=f"{synth.NAMES[type_id]} {mkn} sliced")
    assert np.array_equal(bits(got), bits(q.matmul_t(mkn, lhs)))
