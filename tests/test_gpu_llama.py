"""The device-resident decode step against a plain torch f32 model over the same (decoded) weights."""
import numpy as np
import pytest

import oracle
from joshua_b200 import synth
from joshua_b200.llama import LlamaConfig, LlamaDecoder

pytestmark = pytest.mark.gpu


def torch_reference(dec, tokens_in):
    """f32 torch model: returns the logits of every step when fed `tokens_in` (batch 1)."""
    import torch

    c = dec.cfg
    W = {name: torch.from_numpy(oracle.dequantize(dec.wtype, raw[:-16].cpu().numpy(), two_step=True)).cuda()
         for name, raw in dec._raw.items()}
    shape = {"token_embd": (c.vocab, c.hidden), "output": (c.vocab, c.hidden)}
    for l in range(c.layers):
        shape.update({f"l{l}.wqkv": (c.qkv_rows, c.hidden), f"l{l}.wo": (c.hidden, c.q_heads * c.head_dim),
                      f"l{l}.w_gate": (c.ffn, c.hidden), f"l{l}.w_up": (c.ffn, c.hidden),
                      f"l{l}.w_down": (c.hidden, c.ffn)})
    W = {k: v.reshape(shape[k]).double() for k, v in W.items()}

    def rms(x, w):
        return x / torch.sqrt((x * x).mean() + c.eps) * w.double()

    def rope(v, p):
        half = c.head_dim // 2
        i = torch.arange(half, device="cuda", dtype=torch.float64)
        ang = p * c.rope_theta ** (-2.0 * i / c.head_dim)
        a, b = v[..., :half], v[..., half:]
        return torch.cat([a * torch.cos(ang) - b * torch.sin(ang), a * torch.sin(ang) + b * torch.cos(ang)], dim=-1)

    K = [[] for _ in range(c.layers)]
    V = [[] for _ in range(c.layers)]
    out = []
    for p, tok in enumerate(tokens_in):
        x = W["token_embd"][tok]
        for l, ly in enumerate(dec.layers):
            xn = rms(x, ly["attn_norm"])
            qkv = W[f"l{l}.wqkv"] @ xn
            nq, nkv, hd = c.q_heads, c.kv_heads, c.head_dim
            q = rope(qkv[: nq * hd].reshape(nq, hd), p)
            k = rope(qkv[nq * hd:(nq + nkv) * hd].reshape(nkv, hd), p)
            v = qkv[(nq + nkv) * hd:].reshape(nkv, hd)
            K[l].append(k)
            V[l].append(v)
            Kt, Vt = torch.stack(K[l], 1), torch.stack(V[l], 1)  # [nkv, ctx, hd]
            rep = nq // nkv
            att = torch.einsum("hd,hcd->hc", q, Kt.repeat_interleave(rep, 0)) / np.sqrt(hd)
            att = torch.softmax(att, dim=-1)
            a = torch.einsum("hc,hcd->hd", att, Vt.repeat_interleave(rep, 0)).reshape(-1)
            x1 = x + W[f"l{l}.wo"] @ a
            xn2 = rms(x1, ly["ffn_norm"])
            g, u = W[f"l{l}.w_gate"] @ xn2, W[f"l{l}.w_up"] @ xn2
            x = x1 + W[f"l{l}.w_down"] @ (torch.nn.functional.silu(g) * u)
        out.append((W["output"] @ rms(x, dec.out_norm)).cpu().numpy())
    return out


@pytest.mark.parametrize("wtype", [synth.Q4_K, synth.Q8_0])
def test_decode_steps_match_torch_reference(wtype):
    import torch

    # weights get small scales so that the random model's activations stay O(1)
    def small(name, n, k, s):
        raw = synth.random_weight(wtype, n, k, s).reshape(-1, synth.BLOCK[wtype][1]).copy()
        for off in synth._F16_FIELDS[wtype]:
            sc = raw[:, off:off + 2].copy().view(np.float16).astype(np.float32) * 0.02
            raw[:, off:off + 2] = sc.astype(np.float16).view(np.uint8).reshape(-1, 2)
        return torch.from_numpy(raw.reshape(-1))

    cfg = LlamaConfig(layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=64, ffn=512, vocab=512)
    dec = LlamaDecoder(cfg, torch.device("cuda", 0), batch=1, max_ctx=16, wtype=wtype, seed=3, weights=small)
    fed, got = [], []
    dec.reset(42)
    for step in range(6):
        fed.append(int(dec.token.item()))
        dec.step()
        torch.cuda.synchronize()
        got.append(dec.logits[0].cpu().numpy().copy())
    assert int(dec.pos.item()) == 6 and int(dec.bad.item()) == 0
    want = torch_reference(dec, fed)
    for step in range(6):
        scale = max(1.0, float(np.abs(want[step]).max()))
        assert float(np.abs(got[step] - want[step]).max()) <= 2e-3 * scale, step
        # greedy token: last maximal index wins ties (src/engine.rs:2371-2378)
        ref_tok = len(want[step]) - 1 - int(np.argmax(got[step][::-1]))
        nxt = fed[step + 1] if step + 1 < len(fed) else int(dec.token.item())
        assert nxt == ref_tok


def test_argmax_last_index_wins_ties():
    import ctypes

    import torch

    from joshua_b200 import _lib

    logits = torch.zeros(2, 1000, device="cuda")
    logits[0, 17] = 5.0
    logits[0, 903] = 5.0
    logits[1, :] = -1.0
    tok = torch.zeros(2, dtype=torch.int32, device="cuda")
    pos = torch.tensor([3, 9], dtype=torch.int32, device="cuda")
    scratch = torch.empty(_lib.lib().jq_argmax_scratch_bytes(2) // 4 + 1, device="cuda")
    _lib.check(_lib.lib().jq_argmax_dev(logits.data_ptr(), 2, 1000, tok.data_ptr(), pos.data_ptr(),
                                        scratch.data_ptr(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert tok.tolist() == [903, 999] and pos.tolist() == [4, 10]


def _small_weights(wtype):
    import torch

    def small(name, n, k, s):
        raw = synth.random_weight(wtype, n, k, s).reshape(-1, synth.BLOCK[wtype][1]).copy()
        for off in synth._F16_FIELDS[wtype]:
            sc = raw[:, off:off + 2].copy().view(np.float16).astype(np.float32) * 0.02
            raw[:, off:off + 2] = sc.astype(np.float16).view(np.uint8).reshape(-1, 2)
        return torch.from_numpy(raw.reshape(-1))

    return small


@pytest.mark.parametrize("batch", [1, 3])
def test_fused_step_matches_separate_kernels(batch):
    """The five-launch layer (norms and residuals inside the matmuls, one attention kernel) against the same
    step from the separate kernels, over enough positions to span several attention chunks."""
    import torch

    cfg = LlamaConfig(layers=2, hidden=512, q_heads=8, kv_heads=2, head_dim=64, ffn=768, vocab=512)
    mk = _small_weights(synth.Q4_K)
    a = LlamaDecoder(cfg, torch.device("cuda", 0), batch=batch, max_ctx=80, seed=5, weights=mk)
    b = LlamaDecoder(cfg, torch.device("cuda", 0), batch=batch, max_ctx=80, seed=5, weights=mk)
    a.reset(7)
    b.reset(7)
    for step in range(70):
        a.step()
        b.step_unfused()
        torch.cuda.synchronize()
        la, lb = a.logits.cpu().numpy(), b.logits.cpu().numpy()
        scale = max(1.0, float(np.abs(lb).max()))
        assert float(np.abs(la - lb).max()) <= 2e-4 * scale, step
        b.token.copy_(a.token)   # keep both on the same token stream whatever near-ties do
    assert a.pos.tolist() == [70] * batch


@pytest.mark.parametrize("nq,nkv,hd,ctx", [(8, 2, 64, 1), (8, 8, 128, 33), (32, 4, 128, 100), (16, 2, 256, 64),
                                            (32, 8, 128, 128), (4, 2, 64, 65), (16, 2, 128, 127)])
def test_fused_attention_matches_rope_append_attention(nq, nkv, hd, ctx):
    import torch

    from joshua_b200 import _lib

    L = _lib.lib()
    B, max_ctx, theta = 2, 128, 10000.0
    g = torch.Generator(device="cuda").manual_seed(ctx)
    qkv = torch.randn(B, (nq + 2 * nkv) * hd, device="cuda", generator=g)
    ck = torch.randn(B, nkv, max_ctx, hd, device="cuda", generator=g)
    cv = torch.randn(B, nkv, max_ctx, hd, device="cuda", generator=g)
    ck2, cv2 = ck.clone(), cv.clone()
    pos = torch.tensor([ctx - 1, max(0, ctx - 2)], dtype=torch.int32, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    q = torch.empty(B, nq * hd, device="cuda")
    want = torch.empty(B, nq * hd, device="cuda")
    scratch = torch.empty(L.jq_attention_scratch_bytes(B, nq, hd, max_ctx) // 4 + 1, device="cuda")
    _lib.check(L.jq_rope_append_dev(qkv.data_ptr(), pos.data_ptr(), B, nq, nkv, hd, max_ctx, theta, q.data_ptr(),
                                    ck.data_ptr(), cv.data_ptr(), s))
    _lib.check(L.jq_attention_decode_dev(q.data_ptr(), ck.data_ptr(), cv.data_ptr(), pos.data_ptr(), B, nq, nkv, hd,
                                         max_ctx, want.data_ptr(), scratch.data_ptr(), s))
    got = torch.empty(B, nq * hd, device="cuda")
    fscratch = torch.zeros(L.jq_attention_fused_scratch_bytes(B, nq, nkv, hd, max_ctx) // 4 + 1, device="cuda")
    for _ in range(2):   # twice: the arrival counters must come back to zero
        _lib.check(L.jq_attention_fused_dev(qkv.data_ptr(), pos.data_ptr(), B, nq, nkv, hd, max_ctx, theta,
                                            ck2.data_ptr(), cv2.data_ptr(), got.data_ptr(), fscratch.data_ptr(), s))
    torch.cuda.synchronize()
    assert torch.equal(ck, ck2) and torch.equal(cv, cv2)          # same appended rows, bit for bit
    assert float((got - want).abs().max()) <= 2e-5 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("batch,wtype", [(1, synth.Q4_K), (3, synth.Q4_K), (1, synth.Q8_0)])
def test_chain_step_matches_separate_launches(batch, wtype):
    """The persistent chain (one launch for all layers and the head) against the five-launch-per-layer step:
    same kernels' arithmetic operation by operation, so the logits agree to rounding of the norm sums."""
    import torch

    cfg = LlamaConfig(layers=3, hidden=512, q_heads=8, kv_heads=2, head_dim=128, ffn=768, vocab=1000)
    mk = _small_weights(wtype)
    a = LlamaDecoder(cfg, torch.device("cuda", 0), batch=batch, max_ctx=150, wtype=wtype, seed=5, weights=mk)
    b = LlamaDecoder(cfg, torch.device("cuda", 0), batch=batch, max_ctx=150, wtype=wtype, seed=5, weights=mk)
    a.reset(7)
    b.reset(7)
    for step in range(140):
        a.step_chain()
        b.step()
        torch.cuda.synchronize()
        la, lb = a.logits.cpu().numpy(), b.logits.cpu().numpy()
        scale = max(1.0, float(np.abs(lb).max()))
        assert float(np.abs(la - lb).max()) <= 1e-5 * scale, step
        b.token.copy_(a.token)
    assert a.pos.tolist() == [140] * batch
    from joshua_b200.qtensor import default_context
    from joshua_b200 import _lib
    _lib.check(_lib.lib().jq_device_status(default_context(0)._h))


def test_forward_host_matches_device_steps():
    """The model-level call with host buffers (token ids in, logits out) against the device-resident step."""
    import torch

    cfg = LlamaConfig(layers=2, hidden=512, q_heads=8, kv_heads=2, head_dim=64, ffn=768, vocab=700)
    mk = _small_weights(synth.Q4_K)
    a = LlamaDecoder(cfg, torch.device("cuda", 0), batch=2, max_ctx=32, seed=9, weights=mk)
    b = LlamaDecoder(cfg, torch.device("cuda", 0), batch=2, max_ctx=32, seed=9, weights=mk)
    a.reset(3)
    b.reset(3)
    tok = np.array([3, 3], np.int32)
    for step in range(10):
        logits = a.forward_host(tok).copy()
        b.token.copy_(torch.from_numpy(tok).cuda())
        b.step()
        torch.cuda.synchronize()
        assert np.array_equal(logits, b.logits.cpu().numpy()), step
        tok = logits.argmax(axis=1).astype(np.int32)
    assert a.pos.tolist() == [10, 10]
