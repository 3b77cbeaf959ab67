"""Top-1 decode tokens identical over 64 greedy steps: the device decoders against a CPU model built from the oracle.

Both sides run their OWN greedy loop from the same first token (nothing is teacher-forced): the device samples
on the device (`jq_sample_greedy_dev`, the reference's rule incl. its repetition penalty, src/engine.rs:
1214-1294,2339-2378), the CPU model (tests/cpu_model.py) samples from its own logits.  All 64 token ids must be
equal and every step's logits must agree within 1e-3 * max(|b|, 1).  When a step disagrees the failure message
gives the logit margin between the CPU model's best two candidates, which tells a near-tie from a real error.
"""
import numpy as np
import pytest

from joshua_b200 import synth
from joshua_b200.llama import LlamaConfig, LlamaDecoder
from joshua_b200.moe_decoder import MoeDecoder, MoeDecoderConfig
from tests.cpu_model import CpuDecoder, sample

pytestmark = pytest.mark.gpu
STEPS = 64
TOL = 1e-3   # |a - b| <= TOL * max(|b|, 1), src/kquant_dot.rs:846-851


def small_scales(wtype, factor):
    """Raw random blocks whose f16 scales are shrunk so that the random model's activations stay O(1).  For
    Q4_K the minimum scale is set to 7.5 x the scale, which centres the decoded weights (codes 0..15 minus a
    minimum) around zero: a model of all-positive weights falls into a fixed point within a few tokens."""
    import torch

    def make(name, n, k, s):
        raw = synth.random_weight(wtype, n, k, s).reshape(-1, synth.BLOCK[wtype][1]).copy()
        for off in synth._F16_FIELDS[wtype]:
            sc = raw[:, off:off + 2].copy().view(np.float16).astype(np.float32) * factor
            raw[:, off:off + 2] = sc.astype(np.float16).view(np.uint8).reshape(-1, 2)
        if wtype == synth.Q4_K:
            d = raw[:, 0:2].copy().view(np.float16).astype(np.float32)
            raw[:, 2:4] = (d * 7.5).astype(np.float16).view(np.uint8).reshape(-1, 2)
        return torch.from_numpy(raw.reshape(-1))

    return make


def run_greedy(dec, cpus, first_tokens, penalty):
    import torch

    B = dec.batch
    dec.reset(0)
    dec.token.copy_(torch.tensor(first_tokens, dtype=torch.int32))
    dec.repetition_penalty = penalty
    dec.seed_window([])                       # no prompt: the window starts empty
    fed = [list(first_tokens)]
    recent = [[] for _ in range(B)]
    for step in range(STEPS):
        dec.step()
        torch.cuda.synchronize()
        got = dec.logits.cpu().numpy()
        nxt = dec.token.tolist()
        for b in range(B):
            want = cpus[b].step(fed[step][b])
            err = float((np.abs(got[b] - want) / np.maximum(np.abs(want), 1.0)).max())
            ref_tok = sample(want, penalty, recent[b])
            top2 = np.sort(want)[-2:]
            assert err <= TOL, f"step {step} seq {b}: logits differ by {err:.2e}"
            assert nxt[b] == ref_tok, (f"step {step} seq {b}: device token {nxt[b]}, CPU token {ref_tok}, "
                                       f"CPU logit margin {float(top2[1] - top2[0]):.3e}, max logit error {err:.2e}")
            recent[b] = (recent[b] + [ref_tok])[-64:]
        fed.append(nxt)
    dec.check_flags()
    return fed


@pytest.mark.parametrize("penalty", [1.0, 1.1])
def test_llama_shape_64_greedy_steps_identical(penalty):
    """Q4_K, 4 layers, hidden 1024, FFN 14336, two sequences: inputs of 1024 and 14336 columns, so that the
    activation planes are taken from shared memory (k = 1024) and from scratch in global memory (2 x 14336),
    and the two-row form of the decode kernel runs everywhere."""
    import torch

    cfg = LlamaConfig(layers=4, hidden=1024, q_heads=8, kv_heads=2, head_dim=128, ffn=14336, vocab=2048)
    dec = LlamaDecoder(cfg, torch.device("cuda", 0), batch=2, max_ctx=STEPS + 2, wtype=synth.Q4_K, seed=11,
                       weights=small_scales(synth.Q4_K, 0.02))
    fed = run_greedy(dec, [CpuDecoder(dec), CpuDecoder(dec)], [42, 7], penalty)
    if penalty != 1.0:
        assert len({t[0] for t in fed}) > 8      # the penalty keeps the loop moving through the vocabulary


def test_llama_shape_one_sequence_wide_input():
    """One sequence, hidden 4096: the single-row form over inputs of 4096 columns."""
    import torch

    cfg = LlamaConfig(layers=4, hidden=4096, q_heads=32, kv_heads=8, head_dim=128, ffn=1024, vocab=1024)
    dec = LlamaDecoder(cfg, torch.device("cuda", 0), batch=1, max_ctx=STEPS + 2, wtype=synth.Q4_K, seed=12,
                       weights=small_scales(synth.Q4_K, 0.01))
    run_greedy(dec, [CpuDecoder(dec)], [42], 1.1)


@pytest.mark.parametrize("penalty", [1.0, 1.1])
def test_qwen3moe_shape_64_greedy_steps_identical(penalty):
    """Q8_0 attention, Q4_K experts: 4 layers, hidden 1024, 32 experts top-4 of width 512, softmax routing with
    renormalised weights; the CPU side routes with the oracle's router, so a different expert choice on the
    device shows up as a logit error."""
    import torch

    cfg = MoeDecoderConfig(layers=4, hidden=1024, q_heads=16, kv_heads=4, head_dim=64, vocab=2048, n_expert=32,
                           n_used=4, moe_inter=512)
    dec = MoeDecoder(cfg, torch.device("cuda", 0), batch=1, max_ctx=STEPS + 2, attn_type=synth.Q8_0,
                     expert_type=synth.Q4_K, seed=13, weights=small_scales(synth.Q8_0, 0.02),
                     expert_weights=small_scales(synth.Q4_K, 0.05))
    run_greedy(dec, [CpuDecoder(dec)], [42], penalty)
