"""Prefill (many tokens of one sequence in one pass: batched matmuls incl. the tensor-core tile GEMM, rotary
embedding + cache append for all positions, causal attention) against token-by-token decode on the device and
against the CPU model assembled from the oracle - the reference's own prefill == incremental check
(tests/qwen3moe_tests.rs:93-131, 1e-3) - and a model loaded from a GGUF file written by the test."""
import numpy as np
import pytest

from joshua_b200 import gguf, synth
from joshua_b200.llama import LlamaConfig, LlamaDecoder
from joshua_b200.moe_decoder import MoeDecoder, MoeDecoderConfig, moe_from_gguf
from tests.cpu_model import CpuDecoder, sample
from tests.test_gpu_greedy64 import small_scales

pytestmark = pytest.mark.gpu
TOL = 1e-3


def rel_err(got, want):
    return float((np.abs(got - want) / np.maximum(np.abs(want), 1.0)).max())


def check_prefill(make, prompt, follow=4):
    """Prefill of `prompt` on one decoder, the same tokens one by one on a second one: same logits, same next
    token, the same cache rows, and the steps that follow agree too; the last prompt token's logits also match
    the CPU model's."""
    import torch

    a, b = make(), make()
    a.reset(0)
    b.reset(0)
    a.prefill(prompt)
    for t in prompt:
        b.token.fill_(int(t))
        b.step()
    torch.cuda.synchronize()
    a.check_flags()
    la, lb = a.logits.cpu().numpy(), b.logits.cpu().numpy()
    assert rel_err(la, lb) <= TOL
    assert a.pos.tolist() == b.pos.tolist() == [len(prompt)]
    for x, y in zip(a.layers, b.layers):
        n = len(prompt)
        assert float((x["k"][:, :, :n] - y["k"][:, :, :n]).abs().max()) <= TOL * max(1.0, float(y["k"].abs().max()))
        assert float((x["v"][:, :, :n] - y["v"][:, :, :n]).abs().max()) <= TOL * max(1.0, float(y["v"].abs().max()))
    cpu = CpuDecoder(a)
    for t in prompt:
        want = cpu.step(int(t))
    assert rel_err(la[0], want) <= TOL
    assert int(a.token.item()) == sample(want, 1.0, [])
    for _ in range(follow):          # decode continues from the prefilled cache
        tok = int(a.token.item())
        b.token.fill_(tok)
        a.step()
        b.step()
        torch.cuda.synchronize()
        assert rel_err(a.logits.cpu().numpy(), b.logits.cpu().numpy()) <= TOL
        assert rel_err(a.logits.cpu().numpy()[0], cpu.step(tok)) <= TOL


@pytest.mark.parametrize("seq", [1, 37, 150])
def test_dense_prefill_matches_incremental_decode(seq):
    import torch

    cfg = LlamaConfig(layers=2, hidden=512, q_heads=8, kv_heads=2, head_dim=64, ffn=768, vocab=600)
    make = lambda: LlamaDecoder(cfg, torch.device("cuda", 0), batch=1, max_ctx=seq + 8, wtype=synth.Q4_K, seed=21,
                                weights=small_scales(synth.Q4_K, 0.03), qk_norm=(seq == 37))
    check_prefill(make, list(np.random.default_rng(seq).integers(0, cfg.vocab, seq)))


def test_moe_prefill_matches_incremental_decode():
    import torch

    cfg = MoeDecoderConfig(layers=2, hidden=512, q_heads=8, kv_heads=2, head_dim=128, vocab=600, n_expert=16,
                           n_used=4, moe_inter=256)
    make = lambda: MoeDecoder(cfg, torch.device("cuda", 0), batch=1, max_ctx=64, attn_type=synth.Q8_0,
                              expert_type=synth.Q4_K, seed=22, weights=small_scales(synth.Q8_0, 0.03),
                              expert_weights=small_scales(synth.Q4_K, 0.06), qk_norm=True)
    check_prefill(make, list(np.random.default_rng(5).integers(0, cfg.vocab, 40)))


def test_prefill_past_the_cache_is_reported():
    import torch

    cfg = LlamaConfig(layers=1, hidden=256, q_heads=4, kv_heads=2, head_dim=64, ffn=256, vocab=300)
    dec = LlamaDecoder(cfg, torch.device("cuda", 0), batch=1, max_ctx=8, seed=1, weights=small_scales(synth.Q4_K, 0.03))
    dec.reset(0)
    dec.prefill(list(range(9)))
    with pytest.raises(Exception, match="KV cache"):
        dec.check_flags()


def write_tiny_qwen3moe(path, rng):
    """A structurally complete `qwen3moe` file (tensor names and metadata of src/quantized_qwen3_moe.rs:90-146,
    556-743): Q8_0 attention, Q4_K expert banks, a Q6_K output head, f32 norms and router, per-head q / k norms."""
    L, h, nq, nkv, hd, E, K, inter, vocab = 2, 512, 8, 2, 64, 8, 2, 256, 320
    q8, q4 = small_scales(synth.Q8_0, 0.03), small_scales(synth.Q4_K, 0.06)

    def blocks(mk, rows, cols, seed):
        return mk("", rows, cols, seed).numpy().tobytes()

    def q6(rows, cols, seed):
        raw = synth.random_weight(synth.Q6_K, rows, cols, seed).reshape(-1, 210).copy()
        d = raw[:, 208:210].copy().view(np.float16).astype(np.float32) * 0.002
        raw[:, 208:210] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
        return raw.tobytes()

    f32 = lambda a: np.ascontiguousarray(a, dtype=np.float32).tobytes()
    tensors = [("token_embd.weight", (vocab, h), synth.Q8_0, blocks(q8, vocab, h, 1)),
               ("output_norm.weight", (h,), 0, f32(1 + 0.1 * rng.standard_normal(h))),
               ("output.weight", (vocab, h), synth.Q6_K, q6(vocab, h, 2))]
    for l in range(L):
        p, s = f"blk.{l}", 100 * (l + 1)
        tensors += [
            (f"{p}.attn_norm.weight", (h,), 0, f32(1 + 0.1 * rng.standard_normal(h))),
            (f"{p}.ffn_norm.weight", (h,), 0, f32(1 + 0.1 * rng.standard_normal(h))),
            (f"{p}.attn_q_norm.weight", (hd,), 0, f32(1 + 0.1 * rng.standard_normal(hd))),
            (f"{p}.attn_k_norm.weight", (hd,), 0, f32(1 + 0.1 * rng.standard_normal(hd))),
            (f"{p}.attn_q.weight", (nq * hd, h), synth.Q8_0, blocks(q8, nq * hd, h, s + 1)),
            (f"{p}.attn_k.weight", (nkv * hd, h), synth.Q8_0, blocks(q8, nkv * hd, h, s + 2)),
            (f"{p}.attn_v.weight", (nkv * hd, h), synth.Q8_0, blocks(q8, nkv * hd, h, s + 3)),
            (f"{p}.attn_output.weight", (h, nq * hd), synth.Q8_0, blocks(q8, h, nq * hd, s + 4)),
            (f"{p}.ffn_gate_inp.weight", (E, h), 0, f32(0.5 * rng.standard_normal((E, h)))),
            (f"{p}.ffn_gate_exps.weight", (E, inter, h), synth.Q4_K, blocks(q4, E * inter, h, s + 5)),
            (f"{p}.ffn_down_exps.weight", (E, h, inter), synth.Q4_K, blocks(q4, E * h, inter, s + 6)),
            (f"{p}.ffn_up_exps.weight", (E, inter, h), synth.Q4_K, blocks(q4, E * inter, h, s + 7)),
        ]
    a = "qwen3moe"
    meta = {"general.architecture": a, f"{a}.block_count": L, f"{a}.embedding_length": h, f"{a}.context_length": 64,
            f"{a}.attention.head_count": nq, f"{a}.attention.head_count_kv": nkv, f"{a}.attention.key_length": hd,
            f"{a}.attention.layer_norm_rms_epsilon": 1e-6, f"{a}.rope.freq_base": 1000000.0, f"{a}.expert_count": E,
            f"{a}.expert_used_count": K, f"{a}.expert_feed_forward_length": inter}
    gguf.write_gguf(path, meta, tensors)


def test_model_loaded_from_a_gguf_file_decodes_like_the_cpu_model(tmp_path):
    """File -> header -> tensor directory -> expert slicing -> upload -> 24 greedy steps, against the CPU model over
    the very bytes the loader uploaded (mixed block types: the Q6_K head runs on the exact float path)."""
    import torch

    path = tmp_path / "tiny-qwen3moe.gguf"
    write_tiny_qwen3moe(path, np.random.default_rng(3))
    dec = moe_from_gguf(path, torch.device("cuda", 0), batch=1, max_ctx=40)
    c = dec.cfg
    assert (c.layers, c.hidden, c.q_heads, c.kv_heads, c.head_dim, c.n_expert, c.n_used, c.moe_inter, c.vocab) == \
        (2, 512, 8, 2, 64, 8, 2, 256, 320) and dec.qk_norm and abs(c.rope_theta - 1e6) < 1
    # what went to the device is the file's bytes: expert e of a bank starts e * bytes-per-expert into the tensor
    per = synth.tensor_bytes(synth.Q4_K, 256, 512)
    bank = dec.gguf.tensor_bytes("blk.1.ffn_up_exps.weight")
    assert np.array_equal(dec._expert_raw[1][1][:-16].cpu().numpy()[3 * per:4 * per], bank[3 * per:4 * per])
    cpu = CpuDecoder(dec)
    dec.reset(0)
    dec.prefill([5, 17, 300, 42, 9])
    torch.cuda.synchronize()
    for t in [5, 17, 300, 42, 9]:
        want = cpu.step(t)
    assert rel_err(dec.logits.cpu().numpy()[0], want) <= TOL
    tok = int(dec.token.item())
    assert tok == sample(want, 1.0, [])
    for step in range(24):
        dec.step()
        torch.cuda.synchronize()
        want = cpu.step(tok)
        assert rel_err(dec.logits.cpu().numpy()[0], want) <= TOL, step
        nxt = int(dec.token.item())
        assert nxt == sample(want, 1.0, []), step
        tok = nxt
    dec.check_flags()
