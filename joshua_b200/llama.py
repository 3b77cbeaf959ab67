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
                 seed: int = 0, weights=None):
        import torch

        self.torch, self.cfg, self.dev, self.batch, self.max_ctx, self.wtype = torch, cfg, device, batch, max_ctx, wtype
        self.weight_bytes = 0
        h, f32 = cfg.hidden, dict(dtype=torch.float32, device=device)
        gen = torch.Generator(device=device)
        gen.manual_seed(seed)
        mk = weights or (lambda name, n, k, s: synth.random_weight_torch(wtype, n, k, s, device))
        self._raw = {}

        def q(name, n, k, s):
            raw = mk(name, n, k, s)
            raw = torch.cat([raw.to(device), torch.zeros(16, dtype=torch.uint8, device=device)])
            nbytes = synth.tensor_bytes(wtype, n, k)
            self.weight_bytes += nbytes
            self._raw[name] = raw
            return QTensor.from_device(wtype, raw[:nbytes])

        self.embed = q("token_embd", cfg.vocab, h, seed * 7919 + 1)
        self.weight_bytes -= synth.tensor_bytes(wtype, cfg.vocab, h)  # one row is read per token, not the table
        self.layers = []
        for l in range(cfg.layers):
            s0 = seed * 7919 + 100 + l * 10
            self.layers.append(dict(
                attn_norm=1.0 + 0.1 * torch.randn(h, generator=gen, **f32),
                ffn_norm=1.0 + 0.1 * torch.randn(h, generator=gen, **f32),
                wqkv=q(f"l{l}.wqkv", cfg.qkv_rows, h, s0), wo=q(f"l{l}.wo", h, cfg.q_heads * cfg.head_dim, s0 + 1),
                w_gate=q(f"l{l}.w_gate", cfg.ffn, h, s0 + 2), w_up=q(f"l{l}.w_up", cfg.ffn, h, s0 + 3),
                w_down=q(f"l{l}.w_down", h, cfg.ffn, s0 + 4),
                k=torch.zeros(batch, cfg.kv_heads, max_ctx, cfg.head_dim, **f32),
                v=torch.zeros(batch, cfg.kv_heads, max_ctx, cfg.head_dim, **f32)))
        self.out_norm = 1.0 + 0.1 * torch.randn(h, generator=gen, **f32)
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
            check(L.jq_attention_fused_dev(P(self.qkv), P(self.pos), B, c.q_heads, c.kv_heads, c.head_dim,
                                           self.max_ctx, c.rope_theta, P(ly["k"]), P(ly["v"]), P(self.attn),
                                           P(self.att_fused_scratch), P(self.bad_pos), s))
            check(L.jq_matmul_norm_dev(ly["wo"]._h, B, c.q_heads * c.head_dim, h, P(self.attn), None, 0.0, P(self.x),
                                       P(self.x), s))
            self._ffn(ly, s)
        check(L.jq_matmul_norm_dev(self.output._h, B, h, c.vocab, P(self.x), P(self.out_norm), c.eps, None,
                                   P(self.logits), s))
        self._sample(s)

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
        launches); kept as the cross-check of the fused step."""
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
