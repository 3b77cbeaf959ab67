"""Parity at the full sizes of the benchmark configurations, where the oracle cannot compute the whole product
in seconds: a random window of output rows against the oracle on exactly those rows' bytes, linearity in the
activations, run-to-run bit equality, and for the routed-expert layers one token against the oracle's dispatch
over only the experts that token chose."""
import numpy as np
import pytest

import oracle
from joshua_b200 import synth
from tests.gpu_util import assert_close

pytestmark = pytest.mark.gpu

# (format, n, k): the 4096 x 4096 case of every format, and the Llama-8B-shape linears in Q4_K
SHAPES = [(synth.Q8_0, 4096, 4096), (synth.Q2_K, 4096, 4096), (synth.Q4_K, 4096, 4096), (synth.IQ2_XXS, 4096, 4096),
          (synth.MXFP4, 4096, 4096), (synth.Q4_K, 14336, 4096), (synth.Q4_K, 4096, 14336), (synth.Q4_K, 128256, 4096),
          (synth.IQ2_XXS, 2048, 7168), (synth.MXFP4, 2048, 7168)]


def _device_weight(type_id, n, k, seed):
    import torch

    from joshua_b200.qtensor import QTensor

    dev = torch.device("cuda", 0)
    nbytes = synth.tensor_bytes(type_id, n, k)
    raw = torch.cat([synth.random_weight_torch(type_id, n, k, seed, dev), torch.zeros(16, dtype=torch.uint8, device=dev)])
    return QTensor.from_device(type_id, raw[:nbytes]), raw


@pytest.mark.parametrize("type_id,n,k", SHAPES)
@pytest.mark.parametrize("m", [1, 8, 40, 100])
def test_row_window_matches_oracle_and_product_is_linear(type_id, n, k, m):
    import torch

    q, raw = _device_weight(type_id, n, k, seed=n % 977 + k)
    g = torch.Generator(device="cuda").manual_seed(m)
    x1 = torch.randn(m, k, device="cuda", generator=g)
    x2 = torch.randn(m, k, device="cuda", generator=g)
    y1, y2, y12, again = (torch.empty(m, n, device="cuda") for _ in range(4))
    q.matmul_t_dev((m, k, n), x1, y1)
    q.matmul_t_dev((m, k, n), x2, y2)
    q.matmul_t_dev((m, k, n), x1 + x2, y12)
    q.matmul_t_dev((m, k, n), x1, again)
    torch.cuda.synchronize()
    assert torch.equal(y1, again)                                   # run-to-run identical
    # a window of 48 rows that straddles a 16-row tile boundary, against the oracle on those rows' bytes
    row_bytes = synth.tensor_bytes(type_id, 1, k)
    r0 = (n // 3) | 5
    rows = min(48, n - r0)
    window = raw[r0 * row_bytes:(r0 + rows) * row_bytes].cpu().numpy()
    want = oracle.matmul_t(type_id, (m, k, rows), x1.cpu().numpy(), window)
    assert_close(y1[:, r0:r0 + rows].cpu().numpy(), want, what=f"{synth.NAMES[type_id]} {n}x{k} m={m} window")
    # linearity: f(x1 + x2) = f(x1) + f(x2) up to the path's tolerance
    lin = (y1 + y2).cpu().numpy()
    assert_close(y12.cpu().numpy(), lin, tol=2e-3, what="linearity")


CONFIGS = [
    # Qwen3-MoE layer: 128 experts top-8, hidden 2048, inter 768, Q4_K
    dict(name="qwen3moe", type_id=synth.Q4_K, E=128, K=8, h=2048, inter=768),
    # DeepSeek-V3-shape routed experts in IQ2_XXS (256 experts top-8, hidden 7168, inter 2048)
    dict(name="deepseek_iq2xxs", type_id=synth.IQ2_XXS, E=256, K=8, h=7168, inter=2048),
    # MXFP4 grouped experts (384 experts top-8, hidden 7168, inter 2048)
    dict(name="mxfp4_experts", type_id=synth.MXFP4, E=384, K=8, h=7168, inter=2048),
]


@pytest.mark.parametrize("c", CONFIGS, ids=[c["name"] for c in CONFIGS])
@pytest.mark.parametrize("T", [1, 16])
def test_full_size_moe_tokens_match_oracle_on_their_experts(c, T):
    import torch

    from joshua_b200.moe import GATE_SOFTMAX, Moe, MoeConfig
    from joshua_b200.qtensor import QTensor, default_context

    dev = torch.device("cuda", 0)
    t, E, K, h, inter = c["type_id"], c["E"], c["K"], c["h"], c["inter"]
    ctx = default_context(0)
    banks, keep = [], []
    for i, (rows, cols) in enumerate([(inter, h), (inter, h), (h, inter)]):
        nbytes = synth.tensor_bytes(t, E * rows, cols)
        raw = torch.cat([synth.random_weight_torch(t, E * rows, cols, 31 + i, dev), torch.zeros(16, dtype=torch.uint8, device=dev)])
        keep.append(raw)
        banks.append(QTensor.from_device(t, raw[:nbytes], ctx))
    rng = np.random.default_rng(E + T)
    router = rng.standard_normal((E, h)).astype(np.float32) * 0.5
    cfg = MoeConfig(gating=GATE_SOFTMAX, n_expert=E, n_used=K, hidden=h, inter=inter, norm=True)
    layer = Moe(cfg, router, *banks, ctx=ctx)
    x = (rng.standard_normal((T, h)) * 0.02).astype(np.float32)
    y = layer.forward(x)
    assert np.array_equal(y.view(np.uint32), layer.forward(x).view(np.uint32))      # deterministic
    ids, wts = layer.last_routing(T)
    # routing against the oracle (full router, cheap), then the expert outputs of a few tokens against the
    # oracle's dispatch over a bank that holds only the experts the token chose
    ocfg = oracle.moe_cfg(gating=cfg.gating, n_expert=E, n_used=K, hidden=h, inter=inter, norm=True, decode_path=True)
    want_ids, want_w = oracle.moe_route(ocfg, oracle.moe_logits(x, router))
    assert np.array_equal(ids, want_ids)
    assert np.allclose(wts, want_w, rtol=1e-5, atol=1e-7)
    g_bytes, d_bytes = synth.tensor_bytes(t, inter, h), synth.tensor_bytes(t, h, inter)
    for tok in sorted({0, T // 2, T - 1}):
        chosen = [int(e) for e in ids[tok]]
        mini = [torch.cat([keep[0][e * g_bytes:(e + 1) * g_bytes] for e in chosen]).cpu().numpy(),
                torch.cat([keep[1][e * g_bytes:(e + 1) * g_bytes] for e in chosen]).cpu().numpy(),
                torch.cat([keep[2][e * d_bytes:(e + 1) * d_bytes] for e in chosen]).cpu().numpy()]
        mcfg = oracle.moe_cfg(gating=cfg.gating, n_expert=K, n_used=K, hidden=h, inter=inter, norm=True, decode_path=True)
        local = np.arange(K, dtype=np.uint32).reshape(1, K)
        want = oracle.moe_dispatch(mcfg, x[tok:tok + 1], local, wts[tok:tok + 1].astype(np.float32), [t] * 3, mini, None, None)
        # Random blocks at this width give sums of thousands of large terms of both signs: single elements of the
        # result carry f32 summation-order noise far above 1e-3 of their own (small) value in BOTH
        # implementations, so the bound is taken against the row's largest magnitude.
        scale = max(1.0, float(np.abs(want).max()))
        worst = float(np.abs(y[tok:tok + 1] - want).max()) / scale
        assert worst <= 1e-3, f"{c['name']} T={T} token {tok}: {worst:.3e} of the row's largest magnitude {scale:.3e}"
