"""A CPU decode loop assembled from the oracle, for whole-model parity of the device decoders.

Every quantized linear is `oracle.matmul_t` (the restated fused kernels of src/kquant_dot.rs /
src/iq2xxs.rs / src/mxfp4.rs), the routed-expert FFN is `oracle.moe_logits` / `moe_route` / `moe_dispatch`
(src/quantized_qwen3_moe.rs:412-520), the embedding row is the two-step decode `QuantizedType::embedding`
returns (src/mmap_tensor.rs:140-167); norms, rotary embedding and attention are plain float32 numpy in the
order of the loaders' forward (src/quantized_qwen3_moe.rs:297-386,793-819); the sampler is the reference's
greedy rule with its repetition penalty (src/engine.rs:2339-2378, last maximal index on ties).
"""
from __future__ import annotations

import numpy as np

import oracle
from joshua_b200 import synth

F = np.float32


def sample(logits, penalty, recent):
    v = np.asarray(logits, dtype=F).copy()
    if penalty != 1.0:
        p = F(penalty)
        for t in recent:
            if 0 <= t < len(v):
                v[t] = v[t] / p if v[t] > 0 else v[t] * p
    return len(v) - 1 - int(np.argmax(v[::-1]))


class CpuDecoder:
    """Mirror of `LlamaDecoder` / `MoeDecoder` (one sequence) over the same raw weight bytes."""

    def __init__(self, dec):
        c = self.cfg = dec.cfg
        self.wtype = dec.wtype
        self.types = dict(dec._types)
        self.raw = {name: t[:-16].cpu().numpy() for name, t in dec._raw.items()}
        self.norms = [(ly["attn_norm"].cpu().numpy(), ly["ffn_norm"].cpu().numpy()) for ly in dec.layers]
        self.qk_norms = [(ly["q_norm"].cpu().numpy(), ly["k_norm"].cpu().numpy()) if dec.qk_norm else None
                         for ly in dec.layers]
        self.out_norm = dec.out_norm.cpu().numpy()
        self.moe = None
        if hasattr(dec, "routers"):
            self.moe = dict(routers=dec.routers, etypes=[[dec._expert_types[(l, i)] for i in range(3)]
                                                         for l in range(c.layers)],
                            banks=[[b[:-16].cpu().numpy() for b in layer] for layer in dec._expert_raw],
                            cfg=oracle.moe_cfg(gating=0, n_expert=c.n_expert, n_used=c.n_used, hidden=c.hidden,
                                               inter=c.moe_inter, norm=True, decode_path=True))
        self.K = [np.zeros((c.kv_heads, 0, c.head_dim), F) for _ in range(c.layers)]
        self.V = [np.zeros((c.kv_heads, 0, c.head_dim), F) for _ in range(c.layers)]
        self.pos = 0
        self.row_bytes = synth.tensor_bytes(self.types["token_embd"], 1, c.hidden)

    def linear(self, name, x, n, k):
        return oracle.matmul_t(self.types[name], (1, k, n), x.reshape(1, k), self.raw[name])[0]

    def head_norm(self, v, w):
        """Per-head RMS norm over head_dim (Qwen3 q / k norm, src/quantized_qwen3_moe.rs:343-353)."""
        c = self.cfg
        ss = np.sum(v * v, axis=-1, keepdims=True, dtype=F)
        return (v * (F(1.0) / np.sqrt(ss / F(c.head_dim) + F(c.eps))).astype(F) * w).astype(F)

    def rms(self, x, w):
        c = self.cfg
        ss = F(np.sum(x.astype(F) * x.astype(F), dtype=F))
        return (x * F(1.0 / np.sqrt(ss / F(c.hidden) + F(c.eps))) * w).astype(F)

    def rope(self, v, p):
        c = self.cfg
        half = c.head_dim // 2
        i = np.arange(half, dtype=np.float64)
        ang = (p * c.rope_theta ** (-2.0 * i / c.head_dim))
        cs, sn = np.cos(ang).astype(F), np.sin(ang).astype(F)
        a, b = v[..., :half], v[..., half:]
        return np.concatenate([a * cs - b * sn, a * sn + b * cs], axis=-1).astype(F)

    def step(self, tok: int) -> np.ndarray:
        c, p = self.cfg, self.pos
        h, nq, nkv, hd = c.hidden, c.q_heads, c.kv_heads, c.head_dim
        row = self.raw["token_embd"][tok * self.row_bytes:(tok + 1) * self.row_bytes]
        x = oracle.dequantize(self.types["token_embd"], row, two_step=True).astype(F)
        for l in range(c.layers):
            an, fn = self.norms[l]
            qkv = self.linear(f"l{l}.wqkv", self.rms(x, an), c.qkv_rows, h)
            q, k = qkv[: nq * hd].reshape(nq, hd), qkv[nq * hd:(nq + nkv) * hd].reshape(nkv, hd)
            if self.qk_norms[l] is not None:
                q, k = self.head_norm(q, self.qk_norms[l][0]), self.head_norm(k, self.qk_norms[l][1])
            q, k = self.rope(q, p), self.rope(k, p)
            v = qkv[(nq + nkv) * hd:].reshape(nkv, hd)
            self.K[l] = np.concatenate([self.K[l], k[:, None, :]], axis=1)
            self.V[l] = np.concatenate([self.V[l], v[:, None, :]], axis=1)
            rep = nq // nkv
            Kt, Vt = np.repeat(self.K[l], rep, axis=0), np.repeat(self.V[l], rep, axis=0)   # [nq, ctx, hd]
            att = np.einsum("hd,hcd->hc", q, Kt).astype(F) * F(1.0 / np.sqrt(hd))
            att = np.exp(att - att.max(axis=1, keepdims=True)).astype(F)
            att = (att / att.sum(axis=1, keepdims=True, dtype=F)).astype(F)
            a = np.einsum("hc,hcd->hd", att, Vt).astype(F).reshape(-1)
            x = (x + self.linear(f"l{l}.wo", a, h, nq * hd)).astype(F)
            xn = self.rms(x, fn)
            if self.moe is None:
                g = self.linear(f"l{l}.w_gate", xn, c.ffn, h)
                u = self.linear(f"l{l}.w_up", xn, c.ffn, h)
                act = (g / (F(1.0) + np.exp(-g, dtype=F)) * u).astype(F)
                x = (x + self.linear(f"l{l}.w_down", act, h, c.ffn)).astype(F)
            else:
                m = self.moe
                logits = oracle.moe_logits(xn.reshape(1, h), m["routers"][l])
                ids, wts = oracle.moe_route(m["cfg"], logits)
                y = oracle.moe_dispatch(m["cfg"], xn.reshape(1, h), ids, wts, m["etypes"][l], m["banks"][l])
                x = (x + y[0]).astype(F)
        self.pos += 1
        return self.linear("output", self.rms(x, self.out_norm), c.vocab, h)
