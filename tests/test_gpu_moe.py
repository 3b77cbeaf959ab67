"""The MoE layer through the C ABI against the oracle's restatement of the three loaders' `Moe::forward`."""
import numpy as np
import pytest

import oracle
from joshua_b200 import synth
from joshua_b200._lib import JoshuaB200Error
from joshua_b200.moe import GATE_SIGMOID, GATE_SOFTMAX, GATE_SQRT_SOFTPLUS, OOB_SKIP, Moe, MoeConfig
from joshua_b200.qtensor import QTensor
from tests.gpu_util import assert_close, bits

pytestmark = pytest.mark.gpu


def make_banks(type_id, E, h, inter, seed):
    return [synth.random_weight(type_id, E * inter, h, seed), synth.random_weight(type_id, E * inter, h, seed + 1),
            synth.random_weight(type_id, E * h, inter, seed + 2)]


def oracle_forward(cfg, x, router, banks, types, bias=None, shared=None, shared_types=None, forced=None):
    ocfg = oracle.moe_cfg(gating=cfg.gating, n_expert=cfg.n_expert, n_used=cfg.n_used, hidden=cfg.hidden,
                          inter=cfg.inter, n_group=cfg.n_group, topk_group=cfg.topk_group, norm=cfg.norm,
                          renorm_mode=int(cfg.renorm_plus_eps), oob_policy=cfg.oob_policy, decode_path=True,
                          scale=cfg.scale, clamp=cfg.clamp)
    logits = oracle.moe_logits(x, router)
    ids, w = oracle.moe_route(ocfg, logits, bias=bias, forced_ids=forced)
    y = oracle.moe_dispatch(ocfg, x, ids, w, types, banks, shared_types, shared)
    return ids, w, y


def build(cfg, type_id, seed, down_type=None, bias=None, shared_type=None):
    down_type = down_type or type_id
    rng = np.random.default_rng(seed)
    router = rng.standard_normal((cfg.n_expert, cfg.hidden)).astype(np.float32) * 0.5
    banks = [synth.random_weight(type_id, cfg.n_expert * cfg.inter, cfg.hidden, seed),
             synth.random_weight(type_id, cfg.n_expert * cfg.inter, cfg.hidden, seed + 1),
             synth.random_weight(down_type, cfg.n_expert * cfg.hidden, cfg.inter, seed + 2)]
    types = [type_id, type_id, down_type]
    q = [QTensor.from_bytes(t, b) for t, b in zip(types, banks)]
    shared = sq = None
    if shared_type:
        shared = [synth.random_weight(shared_type, cfg.inter, cfg.hidden, seed + 3),
                  synth.random_weight(shared_type, cfg.inter, cfg.hidden, seed + 4),
                  synth.random_weight(shared_type, cfg.hidden, cfg.inter, seed + 5)]
        sq = [QTensor.from_bytes(shared_type, b) for b in shared]
    moe = Moe(cfg, router, q[0], q[1], q[2], bias=bias, shared=sq)
    return moe, router, banks, types, shared


# x is kept small so that expert outputs stay O(1) with the synthetic weight scales
def tokens(T, h, seed):
    return (np.random.default_rng(seed).standard_normal((T, h)) * 0.02).astype(np.float32)


@pytest.mark.parametrize("T", [1, 2, 5, 16, 70, 1100])   # 1100 tokens: the bucketed (one matmul per expert) path
def test_qwen3moe_style(T):
    cfg = MoeConfig(gating=GATE_SOFTMAX, n_expert=16, n_used=4, hidden=512, inter=256, norm=True)
    moe, router, banks, types, _ = build(cfg, synth.Q4_K, seed=7)
    x = tokens(T, cfg.hidden, T)
    ids, w, want = oracle_forward(cfg, x, router, banks, types)
    got = moe.forward(x)
    gids, gw = moe.last_routing(T)
    assert np.array_equal(gids, ids)
    assert np.allclose(gw, w, rtol=1e-5, atol=1e-7)
    assert_close(got, want, what=f"qwen3moe T={T}")


@pytest.mark.parametrize("T", [1, 3, 33, 2100])   # 2100 tokens: bucketed experts + batched shared expert
def test_deepseek2_style_sigmoid_groups_bias_shared(T):
    cfg = MoeConfig(gating=GATE_SIGMOID, n_expert=32, n_used=4, hidden=512, inter=256, n_group=8, topk_group=4,
                    norm=True, scale=2.5)
    bias = (np.random.default_rng(3).standard_normal(32) * 0.1).astype(np.float32)
    moe, router, banks, types, shared = build(cfg, synth.IQ2_XXS, seed=11, down_type=synth.Q8_0, bias=bias,
                                              shared_type=synth.Q8_0)
    x = tokens(T, cfg.hidden, 100 + T)
    ids, w, want = oracle_forward(cfg, x, router, banks, types, bias=bias, shared=shared,
                                  shared_types=[synth.Q8_0] * 3)
    got = moe.forward(x)
    gids, gw = moe.last_routing(T)
    assert np.array_equal(gids, ids)
    assert np.allclose(gw, w, rtol=1e-5, atol=1e-7)
    assert_close(got, want, what=f"deepseek2 T={T}")


def test_deepseek2_softmax_group_max_rule():
    cfg = MoeConfig(gating=GATE_SOFTMAX, n_expert=16, n_used=2, hidden=256, inter=256, n_group=4, topk_group=2,
                    norm=False)
    moe, router, banks, types, _ = build(cfg, synth.Q2_K, seed=5)
    x = tokens(6, cfg.hidden, 9)
    ids, w, want = oracle_forward(cfg, x, router, banks, types)
    got = moe.forward(x)
    assert np.array_equal(moe.last_routing(6)[0], ids)
    assert_close(got, want)


@pytest.mark.parametrize("T", [1, 9])
def test_deepseek4_style_sqrt_softplus_clamp_and_hash_routing(T):
    cfg = MoeConfig(gating=GATE_SQRT_SOFTPLUS, n_expert=16, n_used=4, hidden=512, inter=256, norm=True, scale=1.5,
                    clamp=0.5, oob_policy=OOB_SKIP)
    moe, router, banks, types, _ = build(cfg, synth.MXFP4, seed=21, down_type=synth.Q2_K)
    x = tokens(T, cfg.hidden, 50 + T)
    ids, w, want = oracle_forward(cfg, x, router, banks, types)
    assert np.array_equal(moe.forward(x).shape, want.shape)
    assert_close(moe.forward(x), want, what="deepseek4 top-k")
    forced = np.random.default_rng(T).integers(0, 16, size=(T, 4)).astype(np.uint32)
    _, w2, want2 = oracle_forward(cfg, x, router, banks, types, forced=forced)
    got2 = moe.forward(x, forced_ids=forced)
    gids, gw = moe.last_routing(T)
    assert np.array_equal(gids, forced) and np.allclose(gw, w2, rtol=1e-5)
    assert_close(got2, want2, what="deepseek4 hash routing")


@pytest.mark.parametrize("type_id,n_expert", [(synth.Q4_K, 32), (synth.MXFP4, 32), (synth.Q4_K, 16)])
def test_prefill_form_per_expert_row_counts(type_id, n_expert):
    """From 128 tokens on every expert is placed on the device by its row count: none, below 12 (decode kernel), 12
    and 32 (one narrow tile), 33 and 128 (one wide tile), 129 (a full tile and a narrow rest), 161 (a full tile and a
    wide rest).  Forced ids (the hash-routing mechanism) fix the counts; n_used = 2 so that a token's experts differ.
    With 32 experts the average is below 24 rows (tile GEMM and decode kernel side by side), with 16 above it (every
    expert as tiles)."""
    cfg = MoeConfig(gating=GATE_SOFTMAX, n_expert=n_expert, n_used=2, hidden=512, inter=256, norm=True,
                    oob_policy=OOB_SKIP)
    moe, router, banks, types, _ = build(cfg, type_id, seed=77)
    counts = [0, 1, 11, 12, 32, 33, 128, 129, 161, 5, 7, 40, 13, 31, 2, 3]          # rows per expert, sum even
    total = sum(counts)
    assert total % 2 == 0
    counts = counts + [0] * (n_expert - 16)
    flat = np.repeat(np.arange(n_expert, dtype=np.uint32), counts)
    # pair position i with position i + total / 2: the list is sorted, so a pair never holds one expert twice unless
    # an expert has more than half of all rows (none does)
    forced = np.stack([flat[:total // 2], flat[total // 2:]], axis=1)
    assert (forced[:, 0] != forced[:, 1]).all()
    T = forced.shape[0]
    assert T >= 128
    x = tokens(T, cfg.hidden, 5)
    if type_id == synth.MXFP4:
        # the synthetic MXFP4 scales reach 2^3: keep the outputs O(1), where the bound |a - b| <= 1e-3 max(|b|, 1) is
        # a relative one (sums of terms of size 100 that cancel to less than 1 are beyond any f32 path)
        x = (x * 0.03).astype(np.float32)
    _, w, want = oracle_forward(cfg, x, router, banks, types, forced=forced)
    got = moe.forward(x, forced_ids=forced)
    gids, gw = moe.last_routing(T)
    assert np.array_equal(gids, forced) and np.allclose(gw, w, rtol=1e-5)
    assert float(np.abs(want).max()) > 0.05   # not a comparison of zeros
    assert_close(got, want, what="prefill form, mixed row counts")
    assert np.array_equal(bits(got), bits(moe.forward(x, forced_ids=forced)))   # run-to-run identical


def test_out_of_range_expert_ids():
    base = dict(gating=GATE_SQRT_SOFTPLUS, n_expert=8, n_used=2, hidden=256, inter=256)
    x = tokens(3, 256, 1)
    forced = np.array([[1, 2], [9, 3], [0, 0]], dtype=np.uint32)
    strict, *_ = build(MoeConfig(**base), synth.Q4_K, seed=2)
    with pytest.raises(JoshuaB200Error, match="out of"):
        strict.forward(x, forced_ids=forced)
    cfg = MoeConfig(**base, oob_policy=OOB_SKIP)
    lenient, router, banks, types, _ = build(cfg, synth.Q4_K, seed=2)
    got = lenient.forward(x, forced_ids=forced)
    # the oracle's skip policy applies to the bucketed path; the routing weights still see the bad id as absent
    ocfg = oracle.moe_cfg(gating=cfg.gating, n_expert=8, n_used=2, hidden=256, inter=256, oob_policy=oracle.OOB_SKIP,
                          decode_path=False)
    ids_ok = forced.copy()
    logits = oracle.moe_logits(x, router)
    # weights: the out-of-range slot contributes probability 0 to the renormalisation
    probs = np.sqrt(np.log1p(np.exp(-np.abs(logits))) + np.maximum(logits, 0))
    w = np.zeros((3, 2), np.float32)
    for t in range(3):
        p = np.array([probs[t, e] if e < 8 else 0.0 for e in forced[t]], dtype=np.float32)
        w[t] = p / max(p.sum(), 6.1035156e-5)
    want = oracle.moe_dispatch(ocfg, x, ids_ok, w, types, banks)
    assert_close(got, want)


def test_prefill_equals_decode_path_and_is_deterministic():
    cfg = MoeConfig(gating=GATE_SOFTMAX, n_expert=16, n_used=4, hidden=512, inter=256)
    moe, *_ = build(cfg, synth.Q4_K, seed=31)
    x = tokens(6, cfg.hidden, 77)
    batched = moe.forward(x)
    again = moe.forward(x)
    assert np.array_equal(batched.view(np.uint32), again.view(np.uint32))
    for t in range(6):
        single = moe.forward(x[t:t + 1])
        assert np.all(np.abs(single[0] - batched[t]) <= 1e-4 * np.maximum(np.abs(batched[t]), 1.0))


def test_device_entries_and_expert_rows():
    import torch

    cfg = MoeConfig(gating=GATE_SOFTMAX, n_expert=16, n_used=4, hidden=512, inter=256)
    moe, router, banks, types, _ = build(cfg, synth.Q4_K, seed=41)
    T = 5
    x = tokens(T, cfg.hidden, 5)
    moe.reserve(T, T * cfg.n_used)
    xd = torch.from_numpy(x).cuda()
    yd = torch.empty_like(xd)
    moe.forward_dev(xd, yd)
    torch.cuda.synchronize()
    moe.status()
    _, _, want = oracle_forward(cfg, x, router, banks, types)
    assert_close(yd.cpu().numpy(), want)
    # routing alone, then the expert MLPs over explicit (row, expert) pairs, combined on the caller's side
    ids = torch.empty(T, cfg.n_used, dtype=torch.int32, device="cuda")
    wts = torch.empty(T, cfg.n_used, dtype=torch.float32, device="cuda")
    moe.route_dev(xd, ids, wts)
    rows = xd.repeat_interleave(cfg.n_used, dim=0).contiguous()
    out = torch.empty_like(rows)
    moe.experts_dev(rows, ids.reshape(-1).contiguous(), out)
    y2 = (out.reshape(T, cfg.n_used, cfg.hidden) * wts[:, :, None]).sum(dim=1)
    torch.cuda.synchronize()
    assert_close(y2.cpu().numpy(), want)
    # the measurement entry: the expert matmuls alone over the job list of the last call; it changes no later result
    moe.forward_dev(xd, yd)
    moe.experts_replay_dev(xd)
    moe.experts_replay_dev(xd)
    y3 = torch.empty_like(xd)
    moe.forward_dev(xd, y3)
    torch.cuda.synchronize()
    moe.status()
    assert np.array_equal(bits(y3.cpu().numpy()), bits(yd.cpu().numpy()))


def test_replay_needs_a_previous_call():
    cfg = MoeConfig(gating=GATE_SOFTMAX, n_expert=16, n_used=4, hidden=512, inter=256)
    moe, *_ = build(cfg, synth.Q4_K, seed=42)
    import torch

    with pytest.raises(JoshuaB200Error, match="job list"):
        moe.experts_replay_dev(torch.zeros(1, cfg.hidden, device="cuda"))


def test_create_rejects_bad_banks():
    cfg = MoeConfig(gating=GATE_SOFTMAX, n_expert=4, n_used=2, hidden=256, inter=256)
    g = QTensor.from_bytes(synth.Q4_K, synth.random_weight(synth.Q4_K, 4 * 256, 256, 1))
    short = QTensor.from_bytes(synth.Q4_K, synth.random_weight(synth.Q4_K, 3 * 256, 256, 1))
    router = np.zeros((4, 256), np.float32)
    with pytest.raises(JoshuaB200Error, match="blocks, expected"):
        Moe(cfg, router, g, g, short)
    with pytest.raises(JoshuaB200Error, match="n_used"):
        Moe(MoeConfig(gating=GATE_SOFTMAX, n_expert=4, n_used=5, hidden=256, inter=256), router, g, g, g)


@pytest.mark.parametrize("T", [1, 4, 8, 12])
@pytest.mark.parametrize("shared", [False, True])
def test_forward_with_norm_and_residual_folded_in(T, shared):
    """y = residual + layer(rmsnorm(x)) in place, against the separate norm kernel + plain layer + add; T <= 8
    takes the four-launch decode path (router, routing and jobs in one kernel), T = 12 the general one."""
    import torch

    from joshua_b200 import _lib

    cfg = MoeConfig(gating=GATE_SOFTMAX, n_expert=16, n_used=4, hidden=512, inter=256, norm=True)
    moe, router, banks, types, _ = build(cfg, synth.Q4_K, seed=51, shared_type=synth.Q8_0 if shared else None)
    moe.reserve(T, T * cfg.n_used)
    g = torch.Generator(device="cuda").manual_seed(T)
    x = torch.randn(T, cfg.hidden, device="cuda", generator=g)
    nw = 0.02 * (1.0 + 0.1 * torch.randn(cfg.hidden, device="cuda", generator=g))   # keeps expert outputs O(1)
    L, s = _lib.lib(), torch.cuda.current_stream().cuda_stream
    xn = torch.empty_like(x)
    _lib.check(L.jq_rmsnorm_dev(x.data_ptr(), None, nw.data_ptr(), 1e-6, T, cfg.hidden, None, xn.data_ptr(), s))
    want = torch.empty_like(x)
    moe.forward_dev(xn, want)
    want += x
    got = x.clone()
    for _ in range(2):   # twice: the router kernel's arrival counter must come back to zero
        got.copy_(x)
        _lib.check(L.jq_moe_forward_norm_add_dev(moe._h, got.data_ptr(), T, None, nw.data_ptr(), 1e-6, got.data_ptr(),
                                                 got.data_ptr(), s))
    torch.cuda.synchronize()
    moe.status()
    assert float((got - want).abs().max()) <= 1e-4 * max(1.0, float(want.abs().max()))
