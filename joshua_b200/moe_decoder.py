"""A Qwen3-MoE-shaped decoder: the Llama-style step of `llama.py` with a routed-expert FFN in every layer.

Attention projections are `attn_type` blocks (Q8_0 in the benchmark configuration), expert banks `expert_type`
blocks (Q4_K).  On one GPU a layer's FFN is `Moe.forward_dev`.  With an expert-parallel group the banks are
split over the ranks and the FFN is `ep.ExpertParallelMoe`: every rank decodes its own sequences, routes
locally, and exchanges activation rows with the owners of the chosen experts.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import _lib, synth
from .llama import LlamaConfig, LlamaDecoder
from .moe import GATE_SOFTMAX, OOB_SKIP, Moe, MoeConfig
from .qtensor import QTensor, default_context


@dataclass
class MoeDecoderConfig(LlamaConfig):
    layers: int = 48
    hidden: int = 2048
    q_heads: int = 32
    kv_heads: int = 4
    head_dim: int = 128
    ffn: int = 256          # unused dense width (kept small: no dense FFN weights are built)
    vocab: int = 151936
    rope_theta: float = 1000000.0
    n_expert: int = 128
    n_used: int = 8
    moe_inter: int = 768


class MoeDecoder(LlamaDecoder):
    def __init__(self, cfg: MoeDecoderConfig, device, batch: int = 1, max_ctx: int = 640, attn_type: int = synth.Q8_0,
                 expert_type: int = synth.Q4_K, seed: int = 0, group=None, weights=None, expert_weights=None,
                 norms=None, qk_norm: bool = False, routers=None):
        """`weights(name, rows, cols, seed)` / `expert_weights(name, rows, cols, seed)` may supply the raw blocks
        of the dense linears / of this rank's slice of an expert bank (flat uint8 tensors); the defaults draw
        them on the device.  `seed` must be the same on every rank: dense weights are replicated."""
        import torch
        import torch.distributed as dist

        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self._expert_type = expert_type
        self._dense_ffn = False
        super().__init__(cfg, device, batch=batch, max_ctx=max_ctx, wtype=attn_type, seed=seed, weights=weights,
                         norms=norms, qk_norm=qk_norm)
        mk_expert = expert_weights or (lambda name, rows, cols, s: synth.random_weight_torch(expert_type, rows, cols, s, device))
        self.routers, self._expert_raw = [], []
        ctx = default_context(device.index or 0)
        E, K, h, I = cfg.n_expert, cfg.n_used, cfg.hidden, cfg.moe_inter
        per = E // self.world
        self.ffn_layers = []
        self.expert_bytes = 0
        gen = torch.Generator(device=device)
        for l in range(cfg.layers):
            # router and banks are the same on every rank for the same layer (seeded by layer, not by rank)
            gen.manual_seed(1000 + l)
            router = (torch.randn(E, h, generator=gen, device=device, dtype=torch.float32) * 0.5).cpu().numpy()
            if routers is not None:
                router = np.ascontiguousarray(routers(l), dtype=np.float32)     # [n_expert, hidden]
            banks = []
            for i, (rows, cols) in enumerate([(I, h), (I, h), (h, I)]):
                full_seed = 5000 + l * 8 + i
                # each rank draws only its own experts' blocks; the seed folds in the first local expert
                raw = mk_expert(f"l{l}.experts{i}", per * rows, cols, full_seed * 1000 + self.rank * per)
                et = expert_type
                if isinstance(raw, tuple):
                    et, raw = raw
                raw = torch.cat([raw.to(device), torch.zeros(16, dtype=torch.uint8, device=device)])
                nbytes = synth.tensor_bytes(et, per * rows, cols)
                self.expert_bytes += nbytes
                banks.append((QTensor.from_device(et, raw[:nbytes], ctx), raw))
                self._expert_types = getattr(self, "_expert_types", {})
                self._expert_types[(l, i)] = et
            self.routers.append(router)
            self._expert_raw.append([b[1] for b in banks])
            if self.world == 1:
                layer = Moe(MoeConfig(gating=GATE_SOFTMAX, n_expert=E, n_used=K, hidden=h, inter=I, norm=True),
                            router, banks[0][0], banks[1][0], banks[2][0], ctx=ctx)
                layer.reserve(batch, batch * K)
                self.ffn_layers.append(dict(moe=layer, keep=banks))
            else:
                from .ep import PeerExchange

                if l == 0:
                    self.exchange = PeerExchange(ctx, E, K, h, batch, group=group)
                rl = Moe(MoeConfig(gating=GATE_SOFTMAX, n_expert=E, n_used=K, hidden=h, inter=I, norm=True), router,
                         None, None, None, ctx=ctx)
                el = Moe(MoeConfig(gating=GATE_SOFTMAX, n_expert=per, n_used=1, hidden=h, inter=I, oob_policy=OOB_SKIP),
                         np.zeros((per, h), np.float32), banks[0][0], banks[1][0], banks[2][0], ctx=ctx)
                cap = batch * K * self.world
                rl.reserve(batch, 0)
                el.reserve(cap, cap)
                self.ffn_layers.append(dict(router=rl, experts=el, keep=banks))
        self.launches_per_step = (3 + (4 if self.world == 1 else 6)) * cfg.layers + 4

    def _ffn(self, ly, s) -> None:
        """self.x += MoE(rmsnorm(self.x; ffn_norm)); the residual add rides in the combine kernel."""
        L, c, B, P = _lib.lib(), self.cfg, self.batch, lambda t: t.data_ptr()
        f = self.ffn_layers[self._layer_index[id(ly)]]
        if "moe" in f:
            _lib.check(L.jq_moe_forward_norm_add_dev(f["moe"]._h, P(self.x), B, None, P(ly["ffn_norm"]), c.eps,
                                                     P(self.x), P(self.x), s))
        else:
            self.exchange.forward_dev(f["router"], f["experts"], self.x, self.x, residual=self.x, stream=s,
                                      norm_w=ly["ffn_norm"], eps=c.eps)

    def _has_dense_ffn(self) -> bool:
        return False

    def matmuls_only(self, stream=None) -> None:
        """The quantized matmuls of one step back to back, over the routing the last step left on the device: QKV and
        output projection per layer, the grouped gate/up and down products of the routed experts, the head (the
        kernel-level roofline probe; norms, attention, router and combine are left out)."""
        L, c, B = _lib.lib(), self.cfg, self.batch
        s = self.torch.cuda.current_stream(self.dev).cuda_stream if stream is None else stream
        h, P = c.hidden, lambda t: t.data_ptr()
        if self.world > 1 and getattr(self, "_probe_rows", None) is None:
            self._probe_rows = self.torch.zeros(self.exchange.rows, h, dtype=self.torch.float32, device=self.dev)
        for i, ly in enumerate(self.layers):
            _lib.check(L.jq_matmul_t_dev(ly["wqkv"]._h, B, h, c.qkv_rows, P(self.xn), P(self.qkv), s))
            _lib.check(L.jq_matmul_t_dev(ly["wo"]._h, B, c.q_heads * c.head_dim, h, P(self.attn), P(self.o), s))
            f = self.ffn_layers[i]
            if "moe" in f:
                f["moe"].experts_replay_dev(self.x, stream=s)
            else:
                f["experts"].experts_replay_dev(self._probe_rows, stream=s)
        _lib.check(L.jq_matmul_t_dev(self.output._h, B, h, c.vocab, P(self.xn), P(self.logits), s))

    def step(self, stream=None) -> None:
        if not hasattr(self, "_layer_index"):
            self._layer_index = {id(ly): i for i, ly in enumerate(self.layers)}
        super().step(stream)

    def prefill(self, token_ids, stream=None) -> None:
        if not hasattr(self, "_layer_index"):
            self._layer_index = {id(ly): i for i, ly in enumerate(self.layers)}
        assert self.world == 1, "prefill runs on one GPU (the exchange windows are sized for decode batches)"
        super().prefill(token_ids, stream)

    def _ffn_prefill(self, ly, x, xn, S, s) -> None:
        """x += MoE(rmsnorm(x; ffn_norm)) over S tokens (`Moe::forward` with n_tokens = seq_len)."""
        L, c, P = _lib.lib(), self.cfg, lambda t: t.data_ptr()
        layer = self.ffn_layers[self._layer_index[id(ly)]]["moe"]
        layer.reserve(S, S * c.n_used)
        _lib.check(L.jq_moe_forward_norm_add_dev(layer._h, P(x), S, None, P(ly["ffn_norm"]), c.eps, P(x), P(x), s))

    def expert_bytes_per_token(self) -> int:
        """Expert-bank bytes one token touches: n_used experts x 3 matrices per layer."""
        c = self.cfg
        per_expert = 2 * synth.tensor_bytes(self._expert_type, c.moe_inter, c.hidden) + \
            synth.tensor_bytes(self._expert_type, c.hidden, c.moe_inter)
        return c.layers * c.n_used * per_expert


def moe_from_gguf(path, device, batch: int = 1, max_ctx: int = 640, group=None) -> MoeDecoder:
    """A `qwen3moe` GGUF file as a device decoder (the reference's `GGUFQWenMoE::from_gguf`,
    src/quantized_qwen3_moe.rs:678-790): dense tensors are uploaded whole on every rank, of each expert bank
    `blk.{i}.ffn_{gate,up,down}_exps.weight` ([n_expert, out, in], experts contiguous) a rank uploads only its own
    run of experts; the router `ffn_gate_inp` is decoded to f32 once."""
    import torch
    import torch.distributed as dist

    from .gguf import GgufFile
    from .llama import _gguf_common, _gguf_providers

    f = GgufFile(path)
    arch = f.header.architecture()
    if arch != "qwen3moe":
        raise ValueError(f"expected a qwen3moe file, found `{arch}`")
    md = f.header.metadata
    hp = _gguf_common(f, arch)
    cfg = MoeDecoderConfig(n_expert=int(md[f"{arch}.expert_count"]), n_used=int(md[f"{arch}.expert_used_count"]),
                           moe_inter=int(md[f"{arch}.expert_feed_forward_length"]), **hp)
    weights, norms = _gguf_providers(f, torch)
    world = dist.get_world_size(group) if group is not None else 1
    rank = dist.get_rank(group) if group is not None else 0
    per = cfg.n_expert // world
    bank_names = ["ffn_gate_exps", "ffn_up_exps", "ffn_down_exps"]

    def expert_weights(name, rows, cols, seed):
        layer, part = name.split(".")
        gname = f"blk.{layer[1:]}.{bank_names[int(part[-1])]}.weight"
        return f.info(gname).dtype, torch.from_numpy(f.expert_bytes(gname, rank * per, per).copy())

    dec = MoeDecoder(cfg, device, batch=batch, max_ctx=max_ctx, group=group, weights=weights, norms=norms,
                     expert_weights=expert_weights, qk_norm="blk.0.attn_q_norm.weight" in f.header.tensors,
                     routers=lambda l: f.float_tensor(f"blk.{l}.ffn_gate_inp.weight"))
    dec.gguf = f
    return dec
