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
        ref_tok = len(want[step]) - 1 - int(np.argmax(want[step][::-1]))
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
                                    ck.data_ptr(), cv.data_ptr(), None, s))
    _lib.check(L.jq_attention_decode_dev(q.data_ptr(), ck.data_ptr(), cv.data_ptr(), pos.data_ptr(), B, nq, nkv, hd,
                                         max_ctx, want.data_ptr(), scratch.data_ptr(), None, s))
    got = torch.empty(B, nq * hd, device="cuda")
    fscratch = torch.zeros(L.jq_attention_fused_scratch_bytes(B, nq, nkv, hd, max_ctx) // 4 + 1, device="cuda")
    for _ in range(2):   # twice: the arrival counters must come back to zero
        _lib.check(L.jq_attention_fused_dev(qkv.data_ptr(), pos.data_ptr(), B, nq, nkv, hd, max_ctx, theta,
                                            ck2.data_ptr(), cv2.data_ptr(), got.data_ptr(), fscratch.data_ptr(),
                                            None, s))
    torch.cuda.synchronize()
    assert torch.equal(ck, ck2) and torch.equal(cv, cv2)          # same appended rows, bit for bit
    assert float((got - want).abs().max()) <= 2e-5 * max(1.0, float(want.abs().max()))


def test_positions_beyond_the_cache_store_nothing_and_raise_the_flag():
    """Stepping past max_ctx: the kernels skip the append and the attention for that sequence, the flag is set,
    the memory behind the cache is untouched (the cache is the front part of a larger canary-filled buffer),
    and a negative position is treated the same way.  Nothing faults: the checks skip the access."""
    import torch

    from joshua_b200 import _lib

    L = _lib.lib()
    B, nq, nkv, hd, max_ctx, theta = 2, 8, 2, 64, 8, 10000.0
    cache_elems = B * nkv * max_ctx * hd
    s = torch.cuda.current_stream().cuda_stream
    for bad_value in (max_ctx, max_ctx + 5, -1):
        big_k = torch.full((cache_elems + 4096,), 7.5, device="cuda")
        big_v = torch.full((cache_elems + 4096,), -7.5, device="cuda")
        qkv = torch.randn(B, (nq + 2 * nkv) * hd, device="cuda")
        pos = torch.tensor([3, bad_value], dtype=torch.int32, device="cuda")
        out = torch.full((B, nq * hd), 123.0, device="cuda")
        q = torch.empty(B, nq * hd, device="cuda")
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        fscratch = torch.zeros(L.jq_attention_fused_scratch_bytes(B, nq, nkv, hd, max_ctx) // 4 + 1, device="cuda")
        _lib.check(L.jq_attention_fused_dev(qkv.data_ptr(), pos.data_ptr(), B, nq, nkv, hd, max_ctx, theta,
                                            big_k.data_ptr(), big_v.data_ptr(), out.data_ptr(), fscratch.data_ptr(),
                                            flag.data_ptr(), s))
        torch.cuda.synchronize()
        assert int(flag.item()) == 1
        assert bool((big_k[cache_elems:] == 7.5).all()) and bool((big_v[cache_elems:] == -7.5).all())
        # sequence 1 stored nothing anywhere in its own cache block either; sequence 0 appended at position 3
        k4 = big_k[:cache_elems].view(B, nkv, max_ctx, hd)
        assert bool((k4[1] == 7.5).all()) and not bool((k4[0, :, 3] == 7.5).all())
        assert bool((out[1] == 123.0).all()) and bool(torch.isfinite(out[0]).all()) and not bool((out[0] == 123.0).any())
        assert bool((fscratch[-B * nkv * 2 - 1:] == 0).all())         # arrival counters back at zero
        flag.zero_()
        _lib.check(L.jq_rope_append_dev(qkv.data_ptr(), pos.data_ptr(), B, nq, nkv, hd, max_ctx, theta, q.data_ptr(),
                                        big_k.data_ptr(), big_v.data_ptr(), flag.data_ptr(), s))
        scratch = torch.empty(L.jq_attention_scratch_bytes(B, nq, hd, max_ctx) // 4 + 1, device="cuda")
        _lib.check(L.jq_attention_decode_dev(q.data_ptr(), big_k.data_ptr(), big_v.data_ptr(), pos.data_ptr(), B, nq,
                                             nkv, hd, max_ctx, out.data_ptr(), scratch.data_ptr(), flag.data_ptr(), s))
        torch.cuda.synchronize()
        assert int(flag.item()) == 1
        assert bool((big_k[cache_elems:] == 7.5).all()) and bool((big_v[cache_elems:] == -7.5).all())
        assert bool(torch.isnan(out[1]).all()) and bool(torch.isfinite(out[0]).all())


def test_decoder_reports_a_full_cache():
    import torch

    cfg = LlamaConfig(layers=1, hidden=256, q_heads=4, kv_heads=2, head_dim=64, ffn=256, vocab=256)
    dec = LlamaDecoder(cfg, torch.device("cuda", 0), batch=1, max_ctx=4, seed=1, weights=_small_weights(synth.Q4_K))
    dec.reset(5)
    for _ in range(4):
        dec.step()
    dec.check_flags()
    dec.step()                      # position 4 of a 4-position cache
    with pytest.raises(Exception, match="KV cache"):
        dec.check_flags()
    dec2 = LlamaDecoder(cfg, torch.device("cuda", 0), batch=1, max_ctx=4, seed=1, weights=_small_weights(synth.Q4_K))
    tok = np.array([5], np.int32)
    for _ in range(4):
        dec2.forward_host(tok)
    with pytest.raises(Exception, match="KV cache"):
        dec2.forward_host(tok)


def reference_sample(logits, penalty, recent):
    """sample_token at temperature 0 (src/engine.rs:2339-2378), in float32 like the reference."""
    v = logits.astype(np.float32).copy()
    p = np.float32(penalty)
    if penalty != 1.0:
        for t in recent:
            if 0 <= t < len(v):
                v[t] = v[t] / p if v[t] > 0 else v[t] * p
    return len(v) - 1 - int(np.argmax(v[::-1]))      # the last maximal index


def test_greedy_sampler_with_repetition_penalty_matches_the_reference_rule():
    import torch

    from joshua_b200 import _lib

    L = _lib.lib()
    rng = np.random.default_rng(0)
    rows, vocab, penalty = 3, 5000, 1.1
    s = torch.cuda.current_stream().cuda_stream
    scratch = torch.empty(L.jq_argmax_scratch_bytes(rows) // 4 + 1, device="cuda")
    window = torch.zeros(rows, 64, dtype=torch.int32, device="cuda")
    state = torch.zeros(rows, 2, dtype=torch.int32, device="cuda")
    token = torch.zeros(rows, dtype=torch.int32, device="cuda")
    pos = torch.zeros(rows, dtype=torch.int32, device="cuda")
    recent = [[] for _ in range(rows)]
    for step in range(150):         # runs well past 64 ids: the ring wraps
        base = rng.standard_normal((rows, vocab)).astype(np.float32)
        # a few near-tied leaders per row, several of them recently sampled, so that the penalty decides
        for r in range(rows):
            lead = list(rng.integers(0, vocab, 3)) + recent[r][-3:]
            base[r, lead] = 4.0 + 0.05 * rng.standard_normal(len(lead)).astype(np.float32)
            if step % 7 == 0 and recent[r]:
                base[r, :] = -np.abs(base[r, :])            # all negative: the penalty multiplies
                base[r, recent[r][-1]] = -1e-3
                base[r, (recent[r][-1] + 1) % vocab] = np.float32(-1.05e-3)
        logits = torch.from_numpy(base).cuda()
        _lib.check(L.jq_sample_greedy_dev(logits.data_ptr(), rows, vocab, penalty, window.data_ptr(), state.data_ptr(),
                                          token.data_ptr(), pos.data_ptr(), scratch.data_ptr(), s))
        torch.cuda.synchronize()
        assert torch.equal(logits.cpu(), torch.from_numpy(base))       # the caller's logits are unchanged
        got = token.tolist()
        for r in range(rows):
            want = reference_sample(base[r], penalty, recent[r])
            assert got[r] == want, (step, r, got[r], want)
            recent[r] = (recent[r] + [want])[-64:]
    assert pos.tolist() == [150] * rows
    # duplicates count once per occurrence: an id held three times is divided three times
    base = np.zeros((1, vocab), np.float32)
    base[0, 10], base[0, 20] = 1.30, 1.0
    window[0, :3] = 10
    state[0] = torch.tensor([3, 3], dtype=torch.int32)
    logits = torch.from_numpy(base).cuda()
    _lib.check(L.jq_sample_greedy_dev(logits.data_ptr(), 1, vocab, penalty, window.data_ptr(), state.data_ptr(),
                                      token.data_ptr(), pos.data_ptr(), scratch.data_ptr(), s))
    torch.cuda.synchronize()
    assert int(token[0]) == 20 == reference_sample(base[0], penalty, [10, 10, 10])   # 1.3 / 1.1^3 < 1.0


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
