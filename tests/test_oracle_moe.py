"""The oracle's MoE routing and dispatch.

Restates the routing/dispatch unit tests of the reference
(src/quantized_qwen3_moe.rs:899-928, src/quantized_deepseek2.rs:1258-1310):
routing weights sum to one, the bucketed prefill path equals the single-token
decode path, plus the gating rules of the three loaders.
"""
import numpy as np
import pytest

import oracle
from joshua_b200 import synth


def banks(type_id, E, h, inter, seed):
    g = synth.random_weight(type_id, E * inter, h, seed)
    u = synth.random_weight(type_id, E * inter, h, seed + 1)
    d = synth.random_weight(type_id, E * h, inter, seed + 2)
    return [g, u, d]


def test_softmax_routing_weights_sum_to_one():
    cfg = oracle.moe_cfg(gating=oracle.GATE_SOFTMAX, n_expert=16, n_used=4, hidden=256, inter=256)
    logits = np.random.default_rng(0).standard_normal((5, 16)).astype(np.float32)
    ids, w = oracle.moe_route(cfg, logits)
    assert ids.shape == (5, 4) and np.allclose(w.sum(axis=1), 1.0, atol=1e-6)
    for t in range(5):
        order = np.argsort(-logits[t], kind="stable")[:4]
        assert np.array_equal(ids[t], order)
    cfg2 = oracle.moe_cfg(gating=oracle.GATE_SOFTMAX, n_expert=16, n_used=4, hidden=256, inter=256, norm=False)
    _, w2 = oracle.moe_route(cfg2, logits)
    p = np.exp(logits - logits.max(axis=1, keepdims=True))
    p /= p.sum(axis=1, keepdims=True)
    assert np.allclose(w2, np.take_along_axis(p, ids.astype(np.int64), axis=1), rtol=1e-5)


def test_sigmoid_bias_steers_selection_only_and_group_limit():
    E, K = 16, 4
    cfg = oracle.moe_cfg(gating=oracle.GATE_SIGMOID, n_expert=E, n_used=K, hidden=256, inter=256, n_group=4,
                         topk_group=2, norm=True, scale=2.5)
    rng = np.random.default_rng(1)
    logits = rng.standard_normal((7, E)).astype(np.float32)
    bias = rng.standard_normal(E).astype(np.float32) * 0.1
    ids, w = oracle.moe_route(cfg, logits, bias=bias)
    s = 1.0 / (1.0 + np.exp(-logits.astype(np.float64)))
    for t in range(7):
        sel = s[t] + bias
        gs = np.sort(sel.reshape(4, 4), axis=1)[:, -2:].sum(axis=1)
        keep = np.argsort(-gs, kind="stable")[:2]
        masked = np.full(E, -np.inf)
        for g in keep:
            masked[g * 4 : g * 4 + 4] = sel[g * 4 : g * 4 + 4]
        want = np.argsort(-masked, kind="stable")[:K]
        assert np.array_equal(ids[t], want)
        ww = s[t][want]
        assert np.allclose(w[t], ww / ww.sum() * 2.5, rtol=1e-5)


def test_sqrt_softplus_and_hash_routing():
    E, K = 8, 2
    cfg = oracle.moe_cfg(gating=oracle.GATE_SQRT_SOFTPLUS, n_expert=E, n_used=K, hidden=256, inter=256, scale=1.5)
    logits = np.random.default_rng(2).standard_normal((3, E)).astype(np.float32) * 3
    p = np.sqrt(np.log1p(np.exp(logits.astype(np.float64))))
    ids, w = oracle.moe_route(cfg, logits)
    for t in range(3):
        want = np.argsort(-p[t], kind="stable")[:K]
        assert np.array_equal(ids[t], want)
        assert np.allclose(w[t], p[t][want] / p[t][want].sum() * 1.5, rtol=1e-5)
    forced = np.array([[7, 0], [3, 3], [1, 2]], dtype=np.uint32)
    ids2, w2 = oracle.moe_route(cfg, logits, forced_ids=forced)
    assert np.array_equal(ids2, forced)
    for t in range(3):
        pp = p[t][forced[t].astype(np.int64)]
        assert np.allclose(w2[t], pp / pp.sum() * 1.5, rtol=1e-5)


def test_kimi_renormalisation_uses_plus_eps():
    cfg = oracle.moe_cfg(gating=oracle.GATE_SIGMOID, n_expert=8, n_used=2, hidden=256, inter=256,
                         renorm_mode=oracle.RENORM_PLUS_EPS)
    logits = np.random.default_rng(3).standard_normal((4, 8)).astype(np.float32)
    _, w = oracle.moe_route(cfg, logits)
    assert np.allclose(w.sum(axis=1), 1.0, atol=1e-6)


@pytest.mark.parametrize("type_id", [oracle.Q4_K, oracle.IQ2_XXS, oracle.MXFP4])
def test_prefill_path_equals_decode_path(type_id):
    E, K, h, inter = 8, 2, 256, 256
    cfg = oracle.moe_cfg(gating=oracle.GATE_SOFTMAX, n_expert=E, n_used=K, hidden=h, inter=inter)
    b = banks(type_id, E, h, inter, seed=11)
    rng = np.random.default_rng(4)
    x = rng.standard_normal((3, h)).astype(np.float32) * 0.1
    router = rng.standard_normal((E, h)).astype(np.float32)
    logits = oracle.moe_logits(x, router)
    ids, w = oracle.moe_route(cfg, logits)
    batched = oracle.moe_dispatch(cfg, x, ids, w, [type_id] * 3, b)
    for t in range(3):
        single = oracle.moe_dispatch(cfg, x[t : t + 1], ids[t : t + 1], w[t : t + 1], [type_id] * 3, b)
        assert np.all(np.abs(single[0] - batched[t]) <= 1e-4 * np.maximum(np.abs(batched[t]), 1.0))


def test_dispatch_matches_dense_evaluation_with_shared_expert_and_clamp():
    E, K, h, inter = 4, 2, 256, 512
    t_id = oracle.Q8_0
    cfg = oracle.moe_cfg(gating=oracle.GATE_SIGMOID, n_expert=E, n_used=K, hidden=h, inter=inter, clamp=0.75,
                         oob_policy=oracle.OOB_SKIP, decode_path=False)
    b = banks(t_id, E, h, inter, seed=21)
    sh = banks(t_id, 1, h, inter, seed=31)
    rng = np.random.default_rng(5)
    x = rng.standard_normal((5, h)).astype(np.float32) * 0.05
    ids = rng.integers(0, E, size=(5, K)).astype(np.uint32)
    ids[2, 1] = E + 3  # out of range: silently skipped under OOB_SKIP
    w = rng.uniform(0.1, 1.0, size=(5, K)).astype(np.float32)
    y = oracle.moe_dispatch(cfg, x, ids, w, [t_id] * 3, b, [t_id] * 3, sh)

    def dense(bank_set, e, xs):
        g = oracle.dequantize(t_id, bank_set[0]).reshape(-1, inter, h)[e].astype(np.float64)
        u = oracle.dequantize(t_id, bank_set[1]).reshape(-1, inter, h)[e].astype(np.float64)
        d = oracle.dequantize(t_id, bank_set[2]).reshape(-1, h, inter)[e].astype(np.float64)
        gv = np.minimum(xs @ g.T, 0.75)
        uv = np.clip(xs @ u.T, -0.75, 0.75)
        return ((gv / (1 + np.exp(-gv))) * uv) @ d.T

    want = np.zeros((5, h))
    for t in range(5):
        for s in range(K):
            if ids[t, s] < E:
                want[t] += w[t, s] * dense(b, int(ids[t, s]), x[t].astype(np.float64))
        want[t] += dense(sh, 0, x[t].astype(np.float64))
    assert np.all(np.abs(y - want) <= 1e-3 * np.maximum(np.abs(want), 1.0))
    cfg_err = oracle.moe_cfg(gating=oracle.GATE_SIGMOID, n_expert=E, n_used=K, hidden=h, inter=inter)
    with pytest.raises(oracle.OracleError, match="out of"):
        oracle.moe_dispatch(cfg_err, x, ids, w, [t_id] * 3, b)
