"""A DeepSeek-V2/V3-shaped decoder: multi-head latent attention (MLA) + routed experts with a shared expert.

Host-side model code in the manner of the reference's loader (`ModelWeights` / `Attention::forward` / `Moe::forward`
of src/quantized_deepseek2.rs:422-597): per layer

    xn   = rmsnorm(x; attn_norm)
    q    = Wq_b . rmsnorm(Wq_a . xn; q_a_norm)                       [n_head, qk_nope + qk_rope]
    comp = Wkv_a . xn                                                [kv_lora + qk_rope]
    kv   = Wkv_b . rmsnorm(comp[:kv_lora]; kv_a_norm)                [n_head, qk_nope + v_dim]
    rope (interleaved, YaRN table) on q[..., qk_nope:] and on k_pe = comp[kv_lora:]
    K[pos] = [k_nope | k_pe] per head, V[pos] = v per head           (the per-head cache of :389-401)
    x   += Wo . attention(q, K, V; scale)
    x   += experts(rmsnorm(x; ffn_norm)) + shared expert             (sigmoid scores, selection bias, group limit)

Every step is a launch through the C ABI on one stream; the RMS norms in front of a matmul ride inside it.  With an
expert-parallel group the routed banks are split over the ranks (`ep.PeerExchange`); attention, router and the
shared expert are replicated.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

from . import _lib, synth
from ._lib import check
from .moe import GATE_SIGMOID, OOB_SKIP, Moe, MoeConfig
from .qtensor import QTensor, default_context


@dataclass
class DeepseekConfig:
    layers: int = 8
    hidden: int = 7168
    n_head: int = 128
    q_lora: int = 1536
    kv_lora: int = 512
    qk_nope: int = 128
    qk_rope: int = 64
    v_dim: int = 128
    vocab: int = 129280
    rope_theta: float = 10000.0
    eps: float = 1e-6
    n_expert: int = 256
    n_used: int = 8
    n_group: int = 8
    topk_group: int = 4
    moe_inter: int = 2048
    weights_scale: float = 2.5
    # YaRN (src/quantized_deepseek2.rs:243-300); factor <= 1 = plain rotary embedding
    yarn_factor: float = 1.0
    yarn_orig_ctx: int = 4096
    yarn_mscale_all_dim: float = 0.0

    @property
    def qd(self) -> int:
        return self.qk_nope + self.qk_rope


def yarn_table(cfg: DeepseekConfig):
    """(inv_freq [qk_rope / 2] f32, mscale, softmax_scale) as the reference builds them
    (src/quantized_deepseek2.rs:175-186,226-300)."""
    dim, theta = cfg.qk_rope, np.float32(cfg.rope_theta)
    idx = np.arange(0, dim, 2, dtype=np.float32)
    extra = (np.float32(1.0) / np.power(theta, idx / np.float32(dim))).astype(np.float32)
    scale = 1.0 / math.sqrt(cfg.qd)
    if cfg.yarn_factor <= 1.0:
        return extra, 1.0, scale
    inter = (np.float32(1.0) / (np.float32(cfg.yarn_factor) * np.power(theta, idx / np.float32(dim)))).astype(np.float32)

    def corr(num_rot):
        return dim * math.log(cfg.yarn_orig_ctx / (num_rot * 2.0 * math.pi)) / (2.0 * math.log(cfg.rope_theta))

    low, high = max(math.floor(corr(32.0)), 0.0), min(math.ceil(corr(1.0)), dim - 1.0)
    if abs(low - high) < 1.1920929e-07:
        high += 0.001
    ramp = np.clip((np.arange(dim // 2, dtype=np.float32) - np.float32(low)) / np.float32(high - low), 0.0, 1.0)
    mask = (np.float32(1.0) - ramp).astype(np.float32)
    inv = (inter * (np.float32(1.0) - mask) + extra * mask).astype(np.float32)

    def get_mscale(s, m):
        return 1.0 if s <= 1.0 else 0.1 * m * math.log(s) + 1.0

    mscale = get_mscale(cfg.yarn_factor, cfg.yarn_mscale_all_dim)
    if cfg.yarn_mscale_all_dim != 0.0:
        scale *= mscale * mscale
    return inv, float(mscale), scale


class DeepseekDecoder:
    """Random-init model of `cfg`: routed expert banks as `expert_type` blocks (IQ2_XXS in the benchmark
    configuration), every other matrix as `wtype` (Q8_0).  `weights(name, type id, rows, cols, seed)` may supply raw
    blocks (names: token_embd, output, l{i}.{wq_a, wq_b, wkv_a, wkv_b, wo, sh_gate, sh_up, sh_down, experts0..2})."""

    def __init__(self, cfg: DeepseekConfig, device, batch: int = 1, max_ctx: int = 256, wtype: int = synth.Q8_0,
                 expert_type: int = synth.IQ2_XXS, seed: int = 0, group=None, weights=None):
        import torch
        import torch.distributed as dist

        self.torch, self.cfg, self.dev, self.batch, self.max_ctx = torch, cfg, device, batch, max_ctx
        self.wtype, self.expert_type, self.group = wtype, expert_type, group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        ctx = self.ctx = default_context(device.index or 0)
        c, B, f32 = cfg, batch, dict(dtype=torch.float32, device=device)
        gen = torch.Generator(device=device)
        gen.manual_seed(seed)
        self._raw, self.weight_bytes, self.expert_bytes = {}, 0, 0
        mk = weights or (lambda name, t, n, k, s: synth.random_weight_torch(t, n, k, s, device))

        def q(name, t, n, k, s, count=True):
            raw = torch.cat([mk(name, t, n, k, s).to(device), torch.zeros(16, dtype=torch.uint8, device=device)])
            nbytes = synth.tensor_bytes(t, n, k)
            if count:
                self.weight_bytes += nbytes
            self._raw[name] = raw
            return QTensor.from_device(t, raw[:nbytes], ctx)

        nv = lambda size: 1.0 + 0.1 * torch.randn(size, generator=gen, **f32)
        h, nh = c.hidden, c.n_head
        self.embed = q("token_embd", wtype, c.vocab, h, seed * 7919 + 1, count=False)
        E, K, I = c.n_expert, c.n_used, c.moe_inter
        per = E // self.world
        mcfg = dict(gating=GATE_SIGMOID, n_used=K, hidden=h, inter=I, n_group=c.n_group, topk_group=c.topk_group,
                    norm=True, scale=c.weights_scale)
        self.layers, self.routers, self.biases = [], [], []
        for l in range(c.layers):
            s0 = seed * 7919 + 100 + 20 * l
            ly = dict(
                attn_norm=nv(h), q_a_norm=nv(c.q_lora), kv_a_norm=nv(c.kv_lora), ffn_norm=nv(h),
                wq_a=q(f"l{l}.wq_a", wtype, c.q_lora, h, s0), wq_b=q(f"l{l}.wq_b", wtype, nh * c.qd, c.q_lora, s0 + 1),
                wkv_a=q(f"l{l}.wkv_a", wtype, c.kv_lora + c.qk_rope, h, s0 + 2),
                wkv_b=q(f"l{l}.wkv_b", wtype, nh * (c.qk_nope + c.v_dim), c.kv_lora, s0 + 3),
                wo=q(f"l{l}.wo", wtype, h, nh * c.v_dim, s0 + 4),
                sh_gate=q(f"l{l}.sh_gate", wtype, I, h, s0 + 5), sh_up=q(f"l{l}.sh_up", wtype, I, h, s0 + 6),
                sh_down=q(f"l{l}.sh_down", wtype, h, I, s0 + 7),
                k=torch.zeros(B, nh, max_ctx, c.qd, **f32), v=torch.zeros(B, nh, max_ctx, c.v_dim, **f32))
            gen.manual_seed(1000 + l)     # the same router and bias on every rank
            router = (torch.randn(E, h, generator=gen, **f32) * 0.05).cpu().numpy()
            bias = (torch.randn(E, generator=gen, **f32) * 0.05).cpu().numpy()
            gen.manual_seed(seed * 31 + l + 1)
            banks = [q(f"l{l}.experts{i}", expert_type, per * rows, cols, (s0 + 8 + i) * 1000 + self.rank * per, count=False)
                     for i, (rows, cols) in enumerate([(I, h), (I, h), (h, I)])]
            self.expert_bytes += sum(synth.tensor_bytes(expert_type, per * r, cc) for r, cc in [(I, h), (I, h), (h, I)])
            if self.world == 1:
                ly["moe"] = Moe(MoeConfig(n_expert=E, **mcfg), router, *banks, bias=bias,
                                shared=(ly["sh_gate"], ly["sh_up"], ly["sh_down"]), ctx=ctx)
                ly["moe"].reserve(B, B * K)
            else:
                from .ep import PeerExchange

                if l == 0:
                    self.exchange = PeerExchange(ctx, E, K, h, B, group=group)
                ly["router"] = Moe(MoeConfig(n_expert=E, **mcfg), router, None, None, None, bias=bias, ctx=ctx)
                ly["experts"] = Moe(MoeConfig(gating=GATE_SIGMOID, n_expert=per, n_used=1, hidden=h, inter=I,
                                              oob_policy=OOB_SKIP), np.zeros((per, h), np.float32), *banks, ctx=ctx)
                ly["router"].reserve(B, 0)
                ly["experts"].reserve(B * K * self.world, B * K * self.world)
            ly["banks"] = banks
            self.routers.append(router)
            self.biases.append(bias)
            self.layers.append(ly)
        self.out_norm = nv(h)
        self.output = q("output", wtype, c.vocab, h, seed * 7919 + 2)
        inv, self.mscale, self.softmax_scale = yarn_table(c)
        self.inv_freq = torch.from_numpy(inv).to(device)
        L = _lib.lib()
        self.token = torch.full((B,), 42, dtype=torch.int32, device=device)
        self.pos = torch.zeros(B, dtype=torch.int32, device=device)
        self.bad = torch.zeros(1, dtype=torch.int32, device=device)
        self.bad_pos = torch.zeros(1, dtype=torch.int32, device=device)
        self.x = torch.empty(B, h, **f32)
        self.xs = torch.empty(B, h, **f32)
        self.qa = torch.empty(B, c.q_lora, **f32)
        self.q = torch.empty(B, nh * c.qd, **f32)
        self.comp = torch.empty(B, c.kv_lora + c.qk_rope, **f32)
        self.ckv = torch.empty(B, c.kv_lora, **f32)
        self.kv = torch.empty(B, nh * (c.qk_nope + c.v_dim), **f32)
        self.att = torch.empty(B, nh * c.v_dim, **f32)
        self.act = torch.empty(B, I, **f32)
        self.logits = torch.empty(B, c.vocab, **f32)
        self.att_scratch = torch.empty(L.jq_attention_scratch_bytes(B, nh, c.v_dim, max_ctx) // 4 + 1, **f32)
        self.argmax_scratch = torch.empty(L.jq_argmax_scratch_bytes(B) // 4 + 1, **f32)
        self.launches_per_step = (10 + (5 if self.world == 1 else 9)) * c.layers + 4

    def step(self, stream=None) -> None:
        """One token per sequence: reads self.token / self.pos, writes self.logits and the next self.token."""
        L, c, B, P = _lib.lib(), self.cfg, self.batch, lambda t: t.data_ptr()
        s = self.torch.cuda.current_stream(self.dev).cuda_stream if stream is None else stream
        h, nh = c.hidden, c.n_head
        check(L.jq_embedding_dev(self.embed._h, P(self.token), B, c.vocab, h, P(self.x), P(self.bad), s))
        for ly in self.layers:
            check(L.jq_matmul_norm_dev(ly["wq_a"]._h, B, h, c.q_lora, P(self.x), P(ly["attn_norm"]), c.eps, None, P(self.qa), s))
            check(L.jq_matmul_norm_dev(ly["wq_b"]._h, B, c.q_lora, nh * c.qd, P(self.qa), P(ly["q_a_norm"]), c.eps, None,
                                       P(self.q), s))
            check(L.jq_matmul_norm_dev(ly["wkv_a"]._h, B, h, c.kv_lora + c.qk_rope, P(self.x), P(ly["attn_norm"]), c.eps,
                                       None, P(self.comp), s))
            check(L.jq_rmsnorm_strided_dev(P(self.comp), c.kv_lora + c.qk_rope, P(ly["kv_a_norm"]), c.eps, B, c.kv_lora,
                                           P(self.ckv), s))
            check(L.jq_matmul_t_dev(ly["wkv_b"]._h, B, c.kv_lora, nh * (c.qk_nope + c.v_dim), P(self.ckv), P(self.kv), s))
            check(L.jq_mla_assemble_dev(P(self.q), P(self.comp), P(self.kv), P(self.pos), B, nh, c.qk_nope, c.qk_rope,
                                        c.v_dim, c.kv_lora, self.max_ctx, P(self.inv_freq), self.mscale, P(ly["k"]),
                                        P(ly["v"]), P(self.bad_pos), s))
            check(L.jq_attention_decode_qkv_dev(P(self.q), P(ly["k"]), P(ly["v"]), P(self.pos), B, nh, nh, c.qd, c.v_dim,
                                                self.max_ctx, self.softmax_scale, P(self.att), P(self.att_scratch),
                                                P(self.bad_pos), s))
            check(L.jq_matmul_norm_dev(ly["wo"]._h, B, nh * c.v_dim, h, P(self.att), None, 0.0, P(self.x), P(self.x), s))
            if self.world == 1:
                check(L.jq_moe_forward_norm_add_dev(ly["moe"]._h, P(self.x), B, None, P(ly["ffn_norm"]), c.eps, P(self.x),
                                                    P(self.x), s))
            else:
                # the shared expert is replicated: xs = x + shared(rmsnorm(x)); then x = xs + routed experts
                check(L.jq_matmul_swiglu_norm_dev(ly["sh_gate"]._h, ly["sh_up"]._h, B, h, c.moe_inter, P(self.x),
                                                  P(ly["ffn_norm"]), c.eps, P(self.act), 0.0, s))
                check(L.jq_matmul_norm_dev(ly["sh_down"]._h, B, c.moe_inter, h, P(self.act), None, 0.0, P(self.x),
                                           P(self.xs), s))
                self.exchange.forward_dev(ly["router"], ly["experts"], self.x, self.x, residual=self.xs, stream=s,
                                          norm_w=ly["ffn_norm"], eps=c.eps)
        check(L.jq_matmul_norm_dev(self.output._h, B, h, c.vocab, P(self.x), P(self.out_norm), c.eps, None,
                                   P(self.logits), s))
        check(L.jq_argmax_dev(P(self.logits), B, c.vocab, P(self.token), P(self.pos), P(self.argmax_scratch), s))

    def reset(self, token: int = 42) -> None:
        self.token.fill_(token)
        self.pos.zero_()

    def check_flags(self) -> None:
        if int(self.bad.item()) != 0:
            raise _lib.JoshuaB200Error(_lib.E_INVALID, "embedding id out of range")
        if int(self.bad_pos.item()) != 0:
            raise _lib.JoshuaB200Error(_lib.E_TOO_LARGE, f"a position ran past the KV cache of {self.max_ctx} positions")
        if self.world == 1:
            for ly in self.layers:
                ly["moe"].status()

    def bytes_per_token(self) -> int:
        """Weight bytes one rank reads for one token at batch 1: dense matrices + head + n_used routed experts."""
        c = self.cfg
        per_expert = 2 * synth.tensor_bytes(self.expert_type, c.moe_inter, c.hidden) + \
            synth.tensor_bytes(self.expert_type, c.hidden, c.moe_inter)
        return self.weight_bytes + c.layers * min(c.n_used, c.n_expert // self.world) * per_expert
