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
    assert _lib.lib().jq_ep_create(ctx._h, 0, 1, 16, 4, 512, 8192, ctypes.byref(h)) != 0  # window too large


def test_absent_peer_times_out_and_the_context_stays_usable():
    """Rank 0 of a two-rank layout whose peer never serves its window (loopback: the peer's window is a private
    local allocation, nothing publishes its flags).  With the wait bound cut to a few thousand polls both waits of
    the layer run out, the kernels return, the status is JQ_E_TIMEOUT exactly once, and ordinary work on the
    same context still passes.  No rank dies and nothing waits without a bound."""
    import ctypes

    import torch

    import oracle
    from joshua_b200 import _lib
    from joshua_b200.moe import GATE_SOFTMAX, OOB_SKIP, Moe, MoeConfig
    from joshua_b200.qtensor import QTensor, default_context

    L, ctx = _lib.lib(), default_context(0)
    world, per = 2, E // 2
    rng = np.random.default_rng(11)
    router = rng.standard_normal((E, H)).astype(np.float32) * 0.5
    banks = [QTensor.from_bytes(synth.Q4_K, synth.random_weight(synth.Q4_K, per * INTER, H, 1), ctx),
             QTensor.from_bytes(synth.Q4_K, synth.random_weight(synth.Q4_K, per * INTER, H, 2), ctx),
             QTensor.from_bytes(synth.Q4_K, synth.random_weight(synth.Q4_K, per * H, INTER, 3), ctx)]
    router_layer = Moe(MoeConfig(gating=GATE_SOFTMAX, n_expert=E, n_used=K, hidden=H, inter=INTER), router,
                       None, None, None, ctx=ctx)
    experts = Moe(MoeConfig(gating=GATE_SOFTMAX, n_expert=per, n_used=1, hidden=H, inter=INTER, oob_policy=OOB_SKIP),
                  np.zeros((per, H), np.float32), *banks, ctx=ctx)
    T = 2
    ep = ctypes.c_void_p()
    _lib.check(L.jq_ep_create(ctx._h, 0, world, E, K, H, T, ctypes.byref(ep)))
    try:
        _lib.check(L.jq_ep_connect_loopback(ep))
        _lib.check(L.jq_ep_set_poll_limit(ep, 4000))
        router_layer.reserve(T, 0)
        experts.reserve(world * T * K, world * T * K)
        _lib.check(L.jq_device_status(ctx._h))            # clean before
        x = torch.from_numpy((rng.standard_normal((T, H)) * 0.02).astype(np.float32)).cuda()
        y = torch.zeros_like(x)
        s = torch.cuda.current_stream().cuda_stream
        _lib.check(L.jq_ep_forward_dev(ep, router_layer._h, experts._h, x.data_ptr(), T, None, y.data_ptr(), s))
        torch.cuda.synchronize()                          # returns: the waits were bounded
        assert L.jq_device_status(ctx._h) == _lib.E_TIMEOUT
        assert L.jq_device_status(ctx._h) == _lib.OK      # reported once, then cleared
        assert bool(torch.isfinite(y).all())
    finally:
        L.jq_ep_free(ep)
    # the context still serves ordinary products
    m, k, n = 1, 1024, 256
    raw = synth.random_weight(synth.Q4_K, n, k, seed=5)
    lhs = synth.random_activations(m, k, seed=6)
    got = QTensor.from_bytes(synth.Q4_K, raw, ctx).matmul_t((m, k, n), lhs)
    want = oracle.matmul_t(synth.Q4_K, (m, k, n), lhs, raw)
    assert float((np.abs(got - want) / np.maximum(np.abs(want), 1.0)).max()) <= 1e-3
