"""Expert-parallel MoE on two GPUs against the single-GPU layer (skipped with fewer than two GPUs): the
torch.distributed orchestration over NCCL all-to-all, and the library's own exchange over peer memory."""
import os
import socket
import sys

import numpy as np
import pytest

from tests.conftest import ROOT

pytestmark = pytest.mark.gpu

E, K, H, INTER = 16, 4, 512, 256
TYPE = 12


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist

    from joshua_b200 import synth
    from joshua_b200.ep import ExpertParallelMoe, PeerExchange, cuda_compute
    from joshua_b200.moe import GATE_SOFTMAX, OOB_SKIP, Moe, MoeConfig
    from joshua_b200.qtensor import Context, QTensor

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ctx = Context(rank)
    rng = np.random.default_rng(0)
    router = rng.standard_normal((E, H)).astype(np.float32) * 0.5
    banks = [synth.random_weight(TYPE, E * INTER, H, 1), synth.random_weight(TYPE, E * INTER, H, 2),
             synth.random_weight(TYPE, E * H, INTER, 3)]
    per = E // world
    g_bytes, d_bytes = per * synth.tensor_bytes(TYPE, INTER, H), per * synth.tensor_bytes(TYPE, H, INTER)
    local = [QTensor.from_bytes(TYPE, banks[0][rank * g_bytes:(rank + 1) * g_bytes], ctx),
             QTensor.from_bytes(TYPE, banks[1][rank * g_bytes:(rank + 1) * g_bytes], ctx),
             QTensor.from_bytes(TYPE, banks[2][rank * d_bytes:(rank + 1) * d_bytes], ctx)]
    full = [QTensor.from_bytes(TYPE, b, ctx) for b in banks]
    T = 6 + rank
    gcfg = MoeConfig(gating=GATE_SOFTMAX, n_expert=E, n_used=K, hidden=H, inter=INTER)
    lcfg = MoeConfig(gating=GATE_SOFTMAX, n_expert=per, n_used=1, hidden=H, inter=INTER)
    router_layer = Moe(gcfg, router, None, None, None, ctx=ctx)
    expert_layer = Moe(lcfg, np.zeros((per, H), np.float32), *local, ctx=ctx)
    single = Moe(gcfg, router, *full, ctx=ctx)
    router_layer.reserve(64, 0)
    expert_layer.reserve(64, 64 * K)
    x = (np.random.default_rng(10 + rank).standard_normal((T, H)) * 0.02).astype(np.float32)
    layer = ExpertParallelMoe(E, K, cuda_compute(router_layer, expert_layer))
    y = layer.forward(torch.from_numpy(x).cuda())
    y2 = layer.forward(torch.from_numpy(x).cuda())
    torch.cuda.synchronize()
    expert_layer.status()
    want = single.forward(x)
    # the same layer through the peer-memory exchange: three exchanges in a row over one window
    exchange = PeerExchange(ctx, E, K, H, max_tokens=8)
    skip_cfg = MoeConfig(gating=GATE_SOFTMAX, n_expert=per, n_used=1, hidden=H, inter=INTER, oob_policy=OOB_SKIP)
    peer_experts = Moe(skip_cfg, np.zeros((per, H), np.float32), *local, ctx=ctx)
    peer_experts.reserve(0, exchange.rows)
    xd = torch.from_numpy(x).cuda()
    outs = [torch.empty_like(xd) for _ in range(3)]
    for o in outs:
        exchange.forward_dev(router_layer, peer_experts, xd, o)
    torch.cuda.synchronize()
    peer_experts.status()
    dist.barrier()
    peer_err = float(np.abs(outs[0].cpu().numpy() - want).max() / max(1.0, np.abs(want).max()))
    peer_diff = float(sum((o != outs[0]).sum().item() for o in outs))
    np.save(os.path.join(out_dir, f"ok{rank}.npy"),
            np.array([float(np.abs(y.cpu().numpy() - want).max() / max(1.0, np.abs(want).max())),
                      float((y != y2).sum().item()), peer_err, peer_diff]))
    exchange.close()
    dist.destroy_process_group()


def test_two_gpu_expert_parallel(tmp_path):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        err, diff, peer_err, peer_diff = np.load(tmp_path / f"ok{r}.npy")
        assert err <= 1e-5 and diff == 0
        assert peer_err <= 1e-5 and peer_diff == 0   # and the same bits on every exchange
