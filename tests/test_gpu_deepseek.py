"""The DeepSeek-shaped decoder (multi-head latent attention, sigmoid routing with selection bias and group limit,
shared expert, IQ2_XXS expert banks) against the CPU model assembled from the oracle, greedy tokens included."""
import numpy as np
import pytest

from joshua_b200 import synth
from joshua_b200.deepseek import DeepseekConfig, DeepseekDecoder, yarn_table
from tests.cpu_model import CpuDeepseek, sample

pytestmark = pytest.mark.gpu


def small(factor_by_type):
    import torch

    def make(name, t, n, k, s):
        raw = synth.random_weight(t, n, k, s).reshape(-1, synth.BLOCK[t][1]).copy()
        for off in synth._F16_FIELDS[t]:
            sc = raw[:, off:off + 2].copy().view(np.float16).astype(np.float32) * factor_by_type[t]
            raw[:, off:off + 2] = sc.astype(np.float16).view(np.uint8).reshape(-1, 2)
        return torch.from_numpy(raw.reshape(-1))

    return make


@pytest.mark.parametrize("yarn", [False, True])
def test_mla_moe_decoder_matches_the_cpu_model(yarn):
    import torch

    cfg = DeepseekConfig(layers=2, hidden=512, n_head=4, q_lora=256, kv_lora=256, qk_nope=64, qk_rope=32, v_dim=64,
                         vocab=400, n_expert=16, n_used=4, n_group=4, topk_group=2, moe_inter=256,
                         yarn_factor=40.0 if yarn else 1.0, yarn_orig_ctx=64, yarn_mscale_all_dim=1.0 if yarn else 0.0)
    dec = DeepseekDecoder(cfg, torch.device("cuda", 0), batch=1, max_ctx=40, seed=4,
                          weights=small({synth.Q8_0: 0.03, synth.IQ2_XXS: 0.3}))
    cpu = CpuDeepseek(dec)
    dec.reset(7)
    tok = 7
    for step in range(32):
        dec.step()
        torch.cuda.synchronize()
        want = cpu.step(tok)
        got = dec.logits.cpu().numpy()[0]
        err = float((np.abs(got - want) / np.maximum(np.abs(want), 1.0)).max())
        assert err <= 1e-3, (step, err)
        nxt = int(dec.token.item())
        assert nxt == sample(want, 1.0, []), step
        tok = nxt
    dec.check_flags()


def test_yarn_table_known_values():
    inv, mscale, scale = yarn_table(DeepseekConfig(qk_rope=64, qk_nope=128))
    assert mscale == 1.0 and abs(scale - 1 / np.sqrt(192)) < 1e-12 and inv[0] == 1.0 and inv.shape == (32,)
    assert abs(inv[1] - 10000.0 ** (-2 / 64)) < 1e-7
    inv2, mscale2, scale2 = yarn_table(DeepseekConfig(yarn_factor=40.0, yarn_orig_ctx=4096, yarn_mscale_all_dim=1.0))
    want = 0.1 * np.log(40.0) + 1.0
    assert abs(mscale2 - want) < 1e-6 and abs(scale2 - want * want / np.sqrt(192)) < 1e-6
    assert inv2[0] == inv[0] and abs(inv2[-1] - inv[-1] / 40.0) < 1e-9      # fast dims extrapolate, slow ones interpolate
