"""A Llama-style decoder whose every step runs on the device through the C ABI.

Host-side model code in the manner of the reference's loaders (embedding ->
per layer {RMS norm -> attention -> residual -> RMS norm -> SwiGLU MLP ->
residual} -> norm -> output head -> greedy token; the shape of
`GGUFQWenMoE::forward`, src/quantized_qwen3_moe.rs:793-819, with a dense MLP).
Weights are quantized tensors (`QTensor`); the step is a fixed sequence of
launches on one stream with no host round trip, so it can be captured in a CUDA
graph.  The KV cache is f32 [batch, n_kv, max_ctx, head_dim] per layer.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

from . import _lib, synth
from ._lib import check
from .qtensor import QTensor


@dataclass
class LlamaConfig:
    layers: int = 32
    hidden: int = 4096
    q_heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 128256
    rope_theta: float = 500000.0
    eps: float = 1e-5

    @property
    def qkv_rows(self) -> int:
        return (self.q_heads + 2 * self.kv_heads) * self.head_dim


class LlamaDecoder:
    """Random-init model of `cfg` with every linear (and the embedding) stored as `wtype` blocks."""

    def __init__(self, cfg: LlamaConfig, device, batch: int = 1, max_ctx: int = 640, wtype: int = synth.Q4_K,
                 seed: int = 0, weights=None, norms=None, qk_norm: bool = False):
        """`weights(name, rows, cols, seed)` may supply a linear's raw blocks (a flat uint8 tensor of `wtype`, or a
        pair (type id, tensor) for files that mix block types); `norms(name, size)` a norm vector (f32 tensor).
        Names: token_embd, output, output_norm, l{i}.{wqkv, wo, w_gate, w_up, w_down, attn_norm, ffn_norm, q_norm,
        k_norm}.  `qk_norm` adds the per-head q / k norms of Qwen3 in front of the rotary embedding."""
        import torch

        self.torch, self.cfg, self.dev, self.batch, self.max_ctx, self.wtype = torch, cfg, device, batch, max_ctx, wtype
        self.weight_bytes = 0
        h, f32 = cfg.hidden, dict(dtype=torch.float32, device=device)
        gen = torch.Generator(device=device)
        gen.manual_seed(seed)
        mk = weights or (lambda name, n, k, s: synth.random_weight_torch(wtype, n, k, s, device))
        self._raw = {}

        self._types = {}

        def q(name, n, k, s):
            raw = mk(name, n, k, s)
            t = wtype
            if isinstance(raw, tuple):
                t, raw = raw
            raw = torch.cat([raw.to(device), torch.zeros(16, dtype=torch.uint8, device=device)])
            nbytes = synth.tensor_bytes(t, n, k)
            self.weight_bytes += nbytes
            self._raw[name] = raw
            self._types[name] = t
            return QTensor.from_device(t, raw[:nbytes])

        def nv(name, size):
            if norms is not None:
                return norms(name, size).to(device=device, dtype=torch.float32).contiguous()
            return 1.0 + 0.1 * torch.randn(size, generator=gen, **f32)

        self.embed = q("token_embd", cfg.vocab, h, seed * 7919 + 1)
        self.weight_bytes -= synth.tensor_bytes(self._types["token_embd"], cfg.vocab, h)  # one row is read per token
        self.layers = []
        for l in range(cfg.layers):
            s0 = seed * 7919 + 100 + l * 10
            ly = dict(
                attn_norm=nv(f"l{l}.attn_norm", h), ffn_norm=nv(f"l{l}.ffn_norm", h),
                wqkv=q(f"l{l}.wqkv", cfg.qkv_rows, h, s0), wo=q(f"l{l}.wo", h, cfg.q_heads * cfg.head_dim, s0 + 1),
                k=torch.zeros(batch, cfg.kv_heads, max_ctx, cfg.head_dim, **f32),
                v=torch.zeros(batch, cfg.kv_heads, max_ctx, cfg.head_dim, **f32))
            if self._has_dense_ffn():
                ly.update(w_gate=q(f"l{l}.w_gate", cfg.ffn, h, s0 + 2), w_up=q(f"l{l}.w_up", cfg.ffn, h, s0 + 3),
                          w_down=q(f"l{l}.w_down", h, cfg.ffn, s0 + 4))
            if qk_norm:
                ly.update(q_norm=nv(f"l{l}.q_norm", cfg.head_dim), k_norm=nv(f"l{l}.k_norm", cfg.head_dim))
            self.layers.append(ly)
        self.qk_norm = qk_norm
        self.out_norm = nv("output_norm", h)
        self.output = q("output", cfg.vocab, h, seed * 7919 + 2)
        B = batch
        self.token = torch.full((B,), 42, dtype=torch.int32, device=device)
        self.pos = torch.zeros(B, dtype=torch.int32, device=device)
        self.bad = torch.zeros(1, dtype=torch.int32, device=device)
        self.bad_pos = torch.zeros(1, dtype=torch.int32, device=device)   # a position ran past the KV cache
        # greedy sampling with the reference's repetition penalty (1.0 = plain arg-max) over the last 64 ids
        self.repetition_penalty = 1.0
        self.window = torch.zeros(B, 64, dtype=torch.int32, device=device)
        self.window_state = torch.zeros(B, 2, dtype=torch.int32, device=device)
        self.x = torch.empty(B, h, **f32)
        self.x1 = torch.empty(B, h, **f32)
        self.xn = torch.empty(B, h, **f32)
        self.qkv = torch.empty(B, cfg.qkv_rows, **f32)
        self.q = torch.empty(B, cfg.q_heads * cfg.head_dim, **f32)
        self.attn = torch.empty(B, cfg.q_heads * cfg.head_dim, **f32)
        self.o = torch.empty(B, h, **f32)
        self.act = torch.empty(B, cfg.ffn, **f32)
        self.d = torch.empty(B, h, **f32)
        self.logits = torch.empty(B, cfg.vocab, **f32)
        att_bytes = _lib.lib().jq_attention_scratch_bytes(B, cfg.q_heads, cfg.head_dim, max_ctx)
        self.att_scratch = torch.empty(att_bytes // 4 + 1, **f32)
        fused_bytes = _lib.lib().jq_attention_fused_scratch_bytes(B, cfg.q_heads, cfg.kv_heads, cfg.head_dim, max_ctx)
        self.att_fused_scratch = torch.zeros(fused_bytes // 4 + 1, **f32)   # holds arrival counters: starts at zero
        self.argmax_scratch = torch.empty(_lib.lib().jq_argmax_scratch_bytes(B) // 4 + 1, **f32)
        self.launches_per_step = 5 * cfg.layers + 4
        self.matmuls_per_step = 4 * cfg.layers + 1

    # ── one token ───────────────────────────────────────────────────────
    def step(self, stream=None) -> None:
        """Decode one token per sequence: reads self.token / self.pos, writes self.logits, the next
        self.token and advances self.pos.  Launches only.  Five launches per layer: the RMS norms ride in the
        prologue of the matmul that consumes them, the residual adds in the epilogue of the matmul that
        produces the branch, and rope + cache append + attention + merge are one kernel.  self.x is the
        residual stream, updated in place."""
        L, c, B = _lib.lib(), self.cfg, self.batch
        s = self.torch.cuda.current_stream(self.dev).cuda_stream if stream is None else stream
        h, P = c.hidden, lambda t: t.data_ptr()
        check(L.jq_embedding_dev(self.embed._h, P(self.token), B, c.vocab, h, P(self.x), P(self.bad), s))
        for ly in self.layers:
            check(L.jq_matmul_norm_dev(ly["wqkv"]._h, B, h, c.qkv_rows, P(self.x), P(ly["attn_norm"]), c.eps, None,
                                       P(self.qkv), s))
            check(L.jq_attention_fused_qknorm_dev(P(self.qkv), P(self.pos), B, c.q_heads, c.kv_heads, c.head_dim,
                                                  self.max_ctx, c.rope_theta,
                                                  P(ly["q_norm"]) if self.qk_norm else None,
                                                  P(ly["k_norm"]) if self.qk_norm else None, c.eps, P(ly["k"]),
                                                  P(ly["v"]), P(self.attn), P(self.att_fused_scratch),
                                                  P(self.bad_pos), s))
            check(L.jq_matmul_norm_dev(ly["wo"]._h, B, c.q_heads * c.head_dim, h, P(self.attn), None, 0.0, P(self.x),
                                       P(self.x), s))
            self._ffn(ly, s)
        check(L.jq_matmul_norm_dev(self.output._h, B, h, c.vocab, P(self.x), P(self.out_norm), c.eps, None,
                                   P(self.logits), s))
        self._sample(s)

    def _has_dense_ffn(self) -> bool:
        return True

    # ── prefill: many tokens of one sequence in one pass ────────────────
    def prefill(self, token_ids, stream=None) -> None:
        """`forward(input [1, seq_len], offset)` of the reference's loaders (src/quantized_qwen3_moe.rs:793-819): the
        prompt's tokens in ONE pass from the current position - batched matmuls (the tensor-core tile GEMM above
        64 tokens), rotary embedding + cache append for all positions, causal attention - then the logits of the
        last token, the sampled next token and the advanced position, exactly as `step` leaves them.  One
        sequence (batch 1).  Buffers are allocated per call."""
        torch, L, c, P = self.torch, _lib.lib(), self.cfg, lambda t: t.data_ptr()
        assert self.batch == 1, "prefill handles one sequence"
        s = torch.cuda.current_stream(self.dev).cuda_stream if stream is None else stream
        ids = torch.as_tensor(token_ids, dtype=torch.int32).to(self.dev)
        S, h, f32 = int(ids.numel()), c.hidden, dict(dtype=torch.float32, device=self.dev)
        x, xn = torch.empty(S, h, **f32), torch.empty(S, h, **f32)
        qkv, q = torch.empty(S, c.qkv_rows, **f32), torch.empty(S, c.q_heads * c.head_dim, **f32)
        att, o = torch.empty(S, c.q_heads * c.head_dim, **f32), torch.empty(S, h, **f32)
        check(L.jq_embedding_dev(self.embed._h, P(ids), S, c.vocab, h, P(x), P(self.bad), s))
        for ly in self.layers:
            check(L.jq_rmsnorm_dev(P(x), None, P(ly["attn_norm"]), c.eps, S, h, None, P(xn), s))
            check(L.jq_matmul_t_dev(ly["wqkv"]._h, S, h, c.qkv_rows, P(xn), P(qkv), s))
            check(L.jq_rope_append_prefill_dev(P(qkv), P(self.pos), S, c.q_heads, c.kv_heads, c.head_dim, self.max_ctx,
                                               c.rope_theta, P(ly["q_norm"]) if self.qk_norm else None,
                                               P(ly["k_norm"]) if self.qk_norm else None, c.eps, P(q), P(ly["k"]),
                                               P(ly["v"]), P(self.bad_pos), s))
            check(L.jq_attention_prefill_dev(P(q), P(ly["k"]), P(ly["v"]), P(self.pos), S, c.q_heads, c.kv_heads,
                                             c.head_dim, self.max_ctx, P(att), P(self.bad_pos), s))
            check(L.jq_matmul_t_dev(ly["wo"]._h, S, c.q_heads * c.head_dim, h, P(att), P(o), s))
            check(L.jq_add_dev(P(x), P(o), S * h, P(x), s))
            self._ffn_prefill(ly, x, xn, S, s)
        # the last token's row -> logits, next token; the position moves past the prompt
        self.x.copy_(x[S - 1:S])
        check(L.jq_matmul_norm_dev(self.output._h, 1, h, c.vocab, P(self.x), P(self.out_norm), c.eps, None,
                                   P(self.logits), s))
        self.pos.add_(S - 1)
        self._sample(s)
        self._keep_prefill = (x, xn, qkv, q, att, o, ids)   # alive until the stream has run them

    def _ffn_prefill(self, ly, x, xn, S, s) -> None:
        """x += FFN(rmsnorm(x; ffn_norm)) over S rows: two batched matmuls + SwiGLU, then the down projection."""
        torch, L, c, P = self.torch, _lib.lib(), self.cfg, lambda t: t.data_ptr()
        f32 = dict(dtype=torch.float32, device=self.dev)
        g, u = torch.empty(S, c.ffn, **f32), torch.empty(S, c.ffn, **f32)
        d = torch.empty(S, c.hidden, **f32)
        check(L.jq_rmsnorm_dev(P(x), None, P(ly["ffn_norm"]), c.eps, S, c.hidden, None, P(xn), s))
        check(L.jq_matmul_t_dev(ly["w_gate"]._h, S, c.hidden, c.ffn, P(xn), P(g), s))
        check(L.jq_matmul_t_dev(ly["w_up"]._h, S, c.hidden, c.ffn, P(xn), P(u), s))
        check(L.jq_swiglu_dev(P(g), P(u), S * c.ffn, 0.0, P(g), s))
        check(L.jq_matmul_t_dev(ly["w_down"]._h, S, c.ffn, c.hidden, P(g), P(d), s))
        check(L.jq_add_dev(P(x), P(d), S * c.hidden, P(x), s))
        self._keep_ffn = (g, u, d)

    def _sample(self, s) -> None:
        """Next token of every sequence from self.logits (`sample_token` of src/engine.rs:2339-2378 at
        temperature 0): repetition penalty over the recent-id window, arg-max with the last maximal index
        winning ties, the id pushed into the window, the position advanced."""
        L, c, B, P = _lib.lib(), self.cfg, self.batch, lambda t: t.data_ptr()
        if self.repetition_penalty == 1.0:
            check(L.jq_argmax_dev(P(self.logits), B, c.vocab, P(self.token), P(self.pos), P(self.argmax_scratch), s))
        else:
            check(L.jq_sample_greedy_dev(P(self.logits), B, c.vocab, self.repetition_penalty, P(self.window),
                                         P(self.window_state), P(self.token), P(self.pos), P(self.argmax_scratch), s))

    def seed_window(self, prompt_ids) -> None:
        """Fills the recent-id window with the tail of the prompt, as the reference's decode loop does
        (src/engine.rs:1222-1232)."""
        torch = self.torch
        tail = [int(t) for t in prompt_ids][-64:]
        w = torch.zeros(self.batch, 64, dtype=torch.int32)
        w[:, :len(tail)] = torch.tensor(tail, dtype=torch.int32)
        self.window.copy_(w)
        self.window_state.copy_(torch.tensor([[len(tail), len(tail) % 64]] * self.batch, dtype=torch.int32))

    def check_flags(self) -> None:
        """Raises if a token id was out of range or a position ran past the KV cache (synchronises)."""
        if int(self.bad.item()) != 0:
            raise _lib.JoshuaB200Error(_lib.E_INVALID, "embedding id out of range")
        if int(self.bad_pos.item()) != 0:
            raise _lib.JoshuaB200Error(_lib.E_TOO_LARGE, f"a position ran past the KV cache of {self.max_ctx} positions")

    def step_unfused(self, stream=None) -> None:
        """The same step from the separate kernels (norm, rope, attention partial + merge as their own
        launches); kept as the cross-check of the fused step.  Models without q / k norms only."""
        assert not self.qk_norm
        L, c, B = _lib.lib(), self.cfg, self.batch
        s = self.torch.cuda.current_stream(self.dev).cuda_stream if stream is None else stream
        h, P = c.hidden, lambda t: t.data_ptr()
        check(L.jq_embedding_dev(self.embed._h, P(self.token), B, c.vocab, h, P(self.x), P(self.bad), s))
        for ly in self.layers:
            check(L.jq_rmsnorm_dev(P(self.x), None, P(ly["attn_norm"]), c.eps, B, h, None, P(self.xn), s))
            check(L.jq_matmul_t_dev(ly["wqkv"]._h, B, h, c.qkv_rows, P(self.xn), P(self.qkv), s))
            check(L.jq_rope_append_dev(P(self.qkv), P(self.pos), B, c.q_heads, c.kv_heads, c.head_dim, self.max_ctx,
                                       c.rope_theta, P(self.q), P(ly["k"]), P(ly["v"]), P(self.bad_pos), s))
            check(L.jq_attention_decode_dev(P(self.q), P(ly["k"]), P(ly["v"]), P(self.pos), B, c.q_heads, c.kv_heads,
                                            c.head_dim, self.max_ctx, P(self.attn), P(self.att_scratch), P(self.bad_pos), s))
            check(L.jq_matmul_t_dev(ly["wo"]._h, B, c.q_heads * c.head_dim, h, P(self.attn), P(self.o), s))
            check(L.jq_add_dev(P(self.x), P(self.o), B * h, P(self.x), s))
            self._ffn(ly, s)
        check(L.jq_rmsnorm_dev(P(self.x), None, P(self.out_norm), c.eps, B, h, None, P(self.xn), s))
        check(L.jq_matmul_t_dev(self.output._h, B, h, c.vocab, P(self.xn), P(self.logits), s))
        self._sample(s)

    def _ffn(self, ly, s) -> None:
        """self.x += FFN(rmsnorm(self.x; ffn_norm)): the dense SwiGLU MLP in two launches."""
        L, c, B, P = _lib.lib(), self.cfg, self.batch, lambda t: t.data_ptr()
        check(L.jq_matmul_swiglu_norm_dev(ly["w_gate"]._h, ly["w_up"]._h, B, c.hidden, c.ffn, P(self.x),
                                          P(ly["ffn_norm"]), c.eps, P(self.act), 0.0, s))
        check(L.jq_matmul_norm_dev(ly["w_down"]._h, B, c.ffn, c.hidden, P(self.act), None, 0.0, P(self.x), P(self.x), s))

    def matmuls_only(self, stream=None) -> None:
        """The quantized matmuls of one token back to back (the kernel-level roofline probe)."""
        L, c, B = _lib.lib(), self.cfg, self.batch
        s = self.torch.cuda.current_stream(self.dev).cuda_stream if stream is None else stream
        h, P = c.hidden, lambda t: t.data_ptr()
        for ly in self.layers:
            check(L.jq_matmul_t_dev(ly["wqkv"]._h, B, h, c.qkv_rows, P(self.xn), P(self.qkv), s))
            check(L.jq_matmul_t_dev(ly["wo"]._h, B, c.q_heads * c.head_dim, h, P(self.attn), P(self.o), s))
            check(L.jq_matmul_swiglu_dev(ly["w_gate"]._h, ly["w_up"]._h, B, h, c.ffn, P(self.xn), P(self.act), 0.0, s))
            check(L.jq_matmul_t_dev(ly["w_down"]._h, B, c.ffn, h, P(self.act), P(self.d), s))
        check(L.jq_matmul_t_dev(self.output._h, B, h, c.vocab, P(self.xn), P(self.logits), s))

    def algorithmic_bytes(self) -> int:
        """Weight bytes of the matmuls + their f32 inputs and outputs, per token step."""
        c, B = self.cfg, self.batch
        io = c.layers * 4 * B * ((c.hidden + c.qkv_rows) + (c.q_heads * c.head_dim + c.hidden) +
                                 (c.hidden + c.ffn) + (c.ffn + c.hidden)) + 4 * B * (c.hidden + c.vocab)
        return self.weight_bytes + io

    # ── the model-level call with host buffers ──────────────────────────
    def forward_host(self, token_ids, out_logits=None):
        """`ModelWeights::forward(input_ids, index_pos) -> logits` for one new token per sequence with HOST
        buffers on both sides (the shape of the reference's model call, src/model.rs:362-364): the token ids
        are copied to the device from pinned memory, the step runs (a CUDA graph captured on first use), the
        logits are copied back to pinned memory and the call returns when they have arrived.  Positions
        advance by one per call; `reset` starts a new sequence."""
        torch = self.torch
        if getattr(self, "_host", None) is None:
            stream = torch.cuda.Stream(self.dev)
            tok_pin = torch.empty(self.batch, dtype=torch.int32).pin_memory()
            log_pin = torch.empty(self.batch, self.cfg.vocab, dtype=torch.float32).pin_memory()
            with torch.cuda.stream(stream):
                pos0 = self.pos.clone()
                self.step(stream.cuda_stream)      # warm-up outside the capture (scratch allocation)
                stream.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    self.step(stream.cuda_stream)
                self.pos.copy_(pos0)
                stream.synchronize()
            self._host = (stream, tok_pin, log_pin, graph)
            self._host_calls = int(self.pos.max().item())
        stream, tok_pin, log_pin, graph = self._host
        if self._host_calls >= self.max_ctx:
            raise _lib.JoshuaB200Error(_lib.E_TOO_LARGE, f"the KV cache holds {self.max_ctx} positions; reset() starts a new sequence")
        self._host_calls += 1
        tok_pin.copy_(torch.as_tensor(token_ids, dtype=torch.int32).reshape(self.batch))
        with torch.cuda.stream(stream):
            self.token.copy_(tok_pin, non_blocking=True)
            graph.replay()
            log_pin.copy_(self.logits, non_blocking=True)
            stream.synchronize()
        if out_logits is not None:
            out_logits[...] = log_pin.numpy()
            return out_logits
        return log_pin.numpy()

    def reset(self, token: int = 42) -> None:
        self.token.fill_(token)
        self.pos.zero_()
        self.window.zero_()
        self.window_state.zero_()
        self._host_calls = 0

    def force_token(self, token: int) -> None:
        self.token.fill_(token)


# ── loading a GGUF file ─────────────────────────────────────────────────
def _gguf_common(f, arch: str):
    """Hyper-parameters the reference's loaders read (src/quantized_qwen3_moe.rs:90-146)."""
    md = f.header.metadata

    def get(key, default=None):
        v = md.get(f"{arch}.{key}", default)
        if v is None:
            raise ValueError(f"GGUF metadata `{arch}.{key}` is missing")
        return v

    heads = int(get("attention.head_count"))
    hidden = int(get("embedding_length"))
    return dict(layers=int(get("block_count")), hidden=hidden, q_heads=heads,
                kv_heads=int(get("attention.head_count_kv", heads)),
                head_dim=int(md.get(f"{arch}.attention.key_length", hidden // heads)),
                vocab=int(f.info("token_embd.weight").dims[0]),
                rope_theta=float(get("rope.freq_base", 10000.0)),
                eps=float(get("attention.layer_norm_rms_epsilon", 1e-6)))


def _gguf_providers(f, torch):
    """(weights, norms) callables over a `GgufFile` for the decoders' tensor names.  The fused QKV matrix is the
    q, k and v tensors' rows one after the other, which is only possible when the three share a block type."""
    names = {"wo": "attn_output", "w_gate": "ffn_gate", "w_up": "ffn_up", "w_down": "ffn_down"}

    def tensor(gname):
        t = f.info(gname)
        return t.dtype, torch.from_numpy(f.tensor_bytes(gname).copy())

    def weights(name, rows, cols, seed):
        if name == "token_embd":
            return tensor("token_embd.weight")
        if name == "output":   # tied to the embedding when absent (src/quantized_qwen3_moe.rs:737-743)
            return tensor("output.weight" if "output.weight" in f.header.tensors else "token_embd.weight")
        layer, part = name.split(".")
        p = f"blk.{layer[1:]}"
        if part == "wqkv":
            parts = [tensor(f"{p}.attn_{x}.weight") for x in ("q", "k", "v")]
            if len({t for t, _ in parts}) != 1:
                raise ValueError(f"{p}: attn_q / attn_k / attn_v have different block types; the fused QKV "
                                 "product needs one")
            return parts[0][0], torch.cat([b for _, b in parts])
        return tensor(f"{p}.{names[part]}.weight")

    def norms(name, size):
        gname = {"output_norm": "output_norm.weight"}.get(name)
        if gname is None:
            layer, part = name.split(".")
            gname = f"blk.{layer[1:]}." + {"attn_norm": "attn_norm", "ffn_norm": "ffn_norm", "q_norm": "attn_q_norm",
                                           "k_norm": "attn_k_norm"}[part] + ".weight"
        return torch.from_numpy(f.float_tensor(gname).reshape(-1).copy())

    return weights, norms


def llama_from_gguf(path, device, batch: int = 1, max_ctx: int = 640) -> LlamaDecoder:
    """A dense decoder (architectures `llama`, `qwen2`, `qwen3`) from a GGUF file.  The rotary embedding pairs
    element i with i + head_dim / 2; files of the `llama` architecture are written for the interleaved pairing and
    need their q / k rows permuted back by whoever writes the file."""
    import torch

    from .gguf import GgufFile

    f = GgufFile(path)
    arch = f.header.architecture()
    hp = _gguf_common(f, arch)
    cfg = LlamaConfig(ffn=int(f.header.metadata[f"{arch}.feed_forward_length"]), **hp)
    weights, norms = _gguf_providers(f, torch)
    dec = LlamaDecoder(cfg, device, batch=batch, max_ctx=max_ctx, weights=weights, norms=norms,
                       qk_norm=f"blk.0.attn_q_norm.weight" in f.header.tensors)
    dec.gguf = f
    return dec
