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


class CpuDeepseek:
    """Mirror of `joshua_b200.deepseek.DeepseekDecoder` (one sequence, all experts on one rank): multi-head latent
    attention as src/quantized_deepseek2.rs:422-504 (interleaved rotary embedding on the rope slices, per-head K / V
    rebuilt for the new token and appended) and its routed experts + shared expert (:522-597)."""

    def __init__(self, dec):
        c = self.cfg = dec.cfg
        self.wtype, self.etype = dec.wtype, dec.expert_type
        self.raw = {name: t[:-16].cpu().numpy() for name, t in dec._raw.items()}
        self.norms = [{k: ly[k].cpu().numpy() for k in ("attn_norm", "q_a_norm", "kv_a_norm", "ffn_norm")} for ly in dec.layers]
        self.out_norm = dec.out_norm.cpu().numpy()
        self.routers, self.biases = dec.routers, dec.biases
        self.inv_freq, self.mscale, self.scale = dec.inv_freq.cpu().numpy(), dec.mscale, dec.softmax_scale
        self.mcfg = oracle.moe_cfg(gating=1, n_expert=c.n_expert, n_used=c.n_used, hidden=c.hidden, inter=c.moe_inter,
                                   n_group=c.n_group, topk_group=c.topk_group, norm=True, scale=c.weights_scale,
                                   decode_path=True)
        self.K = [np.zeros((c.n_head, 0, c.qd), F) for _ in range(c.layers)]
        self.V = [np.zeros((c.n_head, 0, c.v_dim), F) for _ in range(c.layers)]
        self.pos = 0
        self.row_bytes = synth.tensor_bytes(self.wtype, 1, c.hidden)

    def linear(self, name, x, n, k):
        return oracle.matmul_t(self.wtype, (1, k, n), x.reshape(1, k), self.raw[name])[0]

    @staticmethod
    def rms(x, w, eps):
        ss = F(np.sum(x * x, dtype=F))
        return (x * F(1.0 / np.sqrt(ss / F(x.size) + F(eps))) * w).astype(F)

    def rope_i(self, v, p):
        """Interleaved pairs (2i, 2i + 1) of the last axis."""
        ang = (F(p) * self.inv_freq).astype(F)
        cs, sn = (np.cos(ang) * F(self.mscale)).astype(F), (np.sin(ang) * F(self.mscale)).astype(F)
        a, b = v[..., 0::2], v[..., 1::2]
        out = np.empty_like(v)
        out[..., 0::2] = a * cs - b * sn
        out[..., 1::2] = a * sn + b * cs
        return out.astype(F)

    def step(self, tok: int) -> np.ndarray:
        c, p = self.cfg, self.pos
        h, nh = c.hidden, c.n_head
        row = self.raw["token_embd"][tok * self.row_bytes:(tok + 1) * self.row_bytes]
        x = oracle.dequantize(self.wtype, row, two_step=True).astype(F)
        for l in range(c.layers):
            nm = self.norms[l]
            xn = self.rms(x, nm["attn_norm"], c.eps)
            qa = self.linear(f"l{l}.wq_a", xn, c.q_lora, h)
            q = self.linear(f"l{l}.wq_b", self.rms(qa, nm["q_a_norm"], c.eps), nh * c.qd, c.q_lora).reshape(nh, c.qd).copy()
            comp = self.linear(f"l{l}.wkv_a", xn, c.kv_lora + c.qk_rope, h)
            kv = self.linear(f"l{l}.wkv_b", self.rms(comp[:c.kv_lora], nm["kv_a_norm"], c.eps),
                             nh * (c.qk_nope + c.v_dim), c.kv_lora).reshape(nh, c.qk_nope + c.v_dim)
            q[:, c.qk_nope:] = self.rope_i(q[:, c.qk_nope:], p)
            k_pe = self.rope_i(comp[c.kv_lora:], p)
            k_new = np.concatenate([kv[:, :c.qk_nope], np.broadcast_to(k_pe, (nh, c.qk_rope))], axis=1).astype(F)
            self.K[l] = np.concatenate([self.K[l], k_new[:, None, :]], axis=1)
            self.V[l] = np.concatenate([self.V[l], kv[:, None, c.qk_nope:]], axis=1)
            att = np.einsum("hd,hcd->hc", q, self.K[l]).astype(F) * F(self.scale)
            att = np.exp(att - att.max(axis=1, keepdims=True)).astype(F)
            att = (att / att.sum(axis=1, keepdims=True, dtype=F)).astype(F)
            a = np.einsum("hc,hcd->hd", att, self.V[l]).astype(F).reshape(-1)
            x = (x + self.linear(f"l{l}.wo", a, h, nh * c.v_dim)).astype(F)
            xn = self.rms(x, nm["ffn_norm"], c.eps).reshape(1, h)
            logits = oracle.moe_logits(xn, self.routers[l])
            ids, wts = oracle.moe_route(self.mcfg, logits, bias=self.biases[l])
            y = oracle.moe_dispatch(self.mcfg, xn, ids, wts, [self.etype] * 3,
                                    [self.raw[f"l{l}.experts{i}"] for i in range(3)], [self.wtype] * 3,
                                    [self.raw[f"l{l}.sh_{n}"] for n in ("gate", "up", "down")])
            x = (x + y[0]).astype(F)
        self.pos += 1
        return self.linear("output", self.rms(x, self.out_norm, c.eps), c.vocab, h)
