"""Expert-parallel orchestration on two CPU ranks (gloo), with the oracle standing in for the CUDA library.

Checks the multi-rank path of `joshua_b200.ep`: pairs are sent to the owner of their expert, computed there,
returned and combined in slot order, and the result equals the single-process layer.
"""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.conftest import ROOT

E, K, H, INTER, T = 8, 2, 256, 256, 5
TYPE = 12  # Q4_K


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs():
    from joshua_b200 import synth

    rng = np.random.default_rng(0)
    router = rng.standard_normal((E, H)).astype(np.float32) * 0.5
    banks = [synth.random_weight(TYPE, E * INTER, H, 1), synth.random_weight(TYPE, E * INTER, H, 2),
             synth.random_weight(TYPE, E * H, INTER, 3)]
    xs = [(np.random.default_rng(10 + r).standard_normal((T + r, H)) * 0.02).astype(np.float32) for r in range(2)]
    return router, banks, xs


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    import oracle
    from joshua_b200.ep import EpCompute, ExpertParallelMoe

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    router, banks, xs = _inputs()
    per = E // world
    elem_g, elem_d = per * INTER * (H // 256) * 144, per * H * (INTER // 256) * 144
    local = [banks[0][rank * elem_g:(rank + 1) * elem_g], banks[1][rank * elem_g:(rank + 1) * elem_g],
             banks[2][rank * elem_d:(rank + 1) * elem_d]]
    gcfg = oracle.moe_cfg(gating=oracle.GATE_SOFTMAX, n_expert=E, n_used=K, hidden=H, inter=INTER)
    lcfg = oracle.moe_cfg(gating=oracle.GATE_SOFTMAX, n_expert=per, n_used=1, hidden=H, inter=INTER,
                          decode_path=False, oob_policy=oracle.OOB_SKIP)

    def route(x):
        ids, w = oracle.moe_route(gcfg, oracle.moe_logits(x.numpy(), router))
        return torch.from_numpy(ids.astype(np.int32)), torch.from_numpy(w)

    def experts(rows, local_ids):
        ones = np.ones((rows.shape[0], 1), np.float32)
        # unused rows of the fixed-capacity exchange carry an out-of-range id and must come back as zeros
        y = oracle.moe_dispatch(lcfg, rows.numpy(), local_ids.numpy().astype(np.uint32).reshape(-1, 1), ones,
                                [TYPE] * 3, local)
        return torch.from_numpy(y)

    layer = ExpertParallelMoe(E, K, EpCompute(route, experts))
    y = layer.forward(torch.from_numpy(xs[rank]))
    np.save(os.path.join(out_dir, f"y{rank}.npy"), y.numpy())
    # the fixed-capacity variant needs the same number of tokens on every rank
    yf = layer.forward_fixed(torch.from_numpy(xs[rank][:T]))
    np.save(os.path.join(out_dir, f"yf{rank}.npy"), yf.numpy())
    np.save(os.path.join(out_dir, f"load{rank}.npy"), np.array([layer.last_load]))
    dist.destroy_process_group()


def test_two_rank_expert_parallel_matches_single_process(tmp_path):
    import oracle

    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    router, banks, xs = _inputs()
    cfg = oracle.moe_cfg(gating=oracle.GATE_SOFTMAX, n_expert=E, n_used=K, hidden=H, inter=INTER,
                         decode_path=True)
    loads = 0
    for r in range(2):
        ids, w = oracle.moe_route(cfg, oracle.moe_logits(xs[r], router))
        want = oracle.moe_dispatch(cfg, xs[r], ids, w, [TYPE] * 3, banks)
        got = np.load(tmp_path / f"y{r}.npy")
        assert np.all(np.abs(got - want) <= 1e-4 * np.maximum(np.abs(want), 1.0))
        loads += int(np.load(tmp_path / f"load{r}.npy")[0])
        got_fixed = np.load(tmp_path / f"yf{r}.npy")
        assert np.all(np.abs(got_fixed - want[:T]) <= 1e-4 * np.maximum(np.abs(want[:T]), 1.0))
    assert loads == sum(x.shape[0] for x in xs) * K  # every pair was computed exactly once
