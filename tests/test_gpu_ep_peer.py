"""The peer-memory exchange with a single rank (its window is its own memory): every kernel of the exchange
runs, in stream order, against the single-GPU MoE layer; also replayed from a CUDA graph."""
import numpy as np
import pytest

from joshua_b200 import synth

pytestmark = pytest.mark.gpu

E, K, H, INTER = 16, 4, 512, 256


@pytest.mark.parametrize("type_id", [synth.Q4_K, synth.Q8_0])
@pytest.mark.parametrize("T", [1, 5, 8])
def test_single_rank_exchange_matches_layer(type_id, T):
    import torch

    from joshua_b200.ep import PeerExchange
    from joshua_b200.moe import GATE_SOFTMAX, OOB_SKIP, Moe, MoeConfig
    from joshua_b200.qtensor import QTensor, default_context

    ctx = default_context(0)
    rng = np.random.default_rng(T)
    router = rng.standard_normal((E, H)).astype(np.float32) * 0.5
    banks = [QTensor.from_bytes(type_id, synth.random_weight(type_id, E * INTER, H, 1), ctx),
             QTensor.from_bytes(type_id, synth.random_weight(type_id, E * INTER, H, 2), ctx),
             QTensor.from_bytes(type_id, synth.random_weight(type_id, E * H, INTER, 3), ctx)]
    single = Moe(MoeConfig(gating=GATE_SOFTMAX, n_expert=E, n_used=K, hidden=H, inter=INTER), router, *banks, ctx=ctx)
    router_layer = Moe(MoeConfig(gating=GATE_SOFTMAX, n_expert=E, n_used=K, hidden=H, inter=INTER), router,
                       None, None, None, ctx=ctx)
    experts = Moe(MoeConfig(gating=GATE_SOFTMAX, n_expert=E, n_used=1, hidden=H, inter=INTER, oob_policy=OOB_SKIP),
                  np.zeros((E, H), np.float32), *banks, ctx=ctx)
    exchange = PeerExchange(ctx, E, K, H, max_tokens=8)
    router_layer.reserve(8, 0)
    experts.reserve(0, exchange.rows)
    x = (rng.standard_normal((T, H)) * 0.02).astype(np.float32)
    want = single.forward(x)
    xd = torch.from_numpy(x).cuda()
    y = torch.empty_like(xd)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for _ in range(2):
            exchange.forward_dev(router_layer, experts, xd, y)
        stream.synchronize()
        eager = y.clone()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            exchange.forward_dev(router_layer, experts, xd, y)
        y.zero_()
        graph.replay()
        graph.replay()
        stream.synchronize()
    experts.status()
    got = eager.cpu().numpy()
    assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max())
    assert torch.equal(y, eager)
    exchange.close()


def test_exchange_rejects_bad_arguments():
    import ctypes

    from joshua_b200 import _lib
    from joshua_b200.qtensor import default_context

    ctx = default_context(0)
    h = ctypes.c_void_p()
    assert _lib.lib().jq_ep_create(ctx._h, 0, 3, 16, 4, 512, 8, ctypes.byref(h)) != 0   # 16 experts over 3 ranks
    assert b"evenly" in _lib.lib().jq_last_error()
    assert _lib.lib().jq_ep_create(ctx._h, 2, 2, 16, 4, 512, 8, ctypes.byref(h)) != 0   # rank out of range
    assert _lib.lib().jq_ep_create(ctx._h, 0, 1, 16, 4, 512, 4096, ctypes.byref(h)) != 0  # window too large
