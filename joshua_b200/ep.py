"""Expert-parallel MoE across the GPUs of one node.

The reference runs in one process on one device; this is the one place the
path shards.  Experts are split contiguously over the ranks of a
`torch.distributed` group (expert e lives on rank e // (E / G), matching the
contiguous [n_expert, out, in] layout of the expert tensors,
src/quantized_qwen3_moe.rs:572-613); router and dense weights are replicated.
Every rank holds its own tokens.  One layer is

    route (local, replicated router)            -> ids, weights        [T, k]
    sort the (token, slot) pairs by owner rank  -> send order
    all-to-all: activation rows + local expert ids to the owners   (dispatch)
    expert MLPs over the received rows          (grouped matmul on the owner)
    all-to-all: outputs back                                        (combine)
    y[t] = sum over slots, in slot order, of w[t, s] * out[t, s]

The summation order does not depend on the number of ranks, so outputs are
the same for 1, 2, 4 or 8 GPUs up to nothing at all (bit-identical).

The exchange needs per-peer row counts on the host (one small all-to-all of
counts and one host read per layer).  `compute` is injected so that the
orchestration can be exercised on CPU ranks (gloo) with a stand-in for the
CUDA library.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch
import torch.distributed as dist


@dataclass
class EpCompute:
    """The two device steps of a layer.

    route(x [T, h]) -> (ids int32 [T, k] global expert ids, wts f32 [T, k])
    experts(rows [R, h], local_ids int32 [R]) -> out [R, h]   (unweighted MLP outputs)
    """

    route: Callable
    experts: Callable


def _exchange_rows(send: torch.Tensor, send_counts: list[int], recv_counts: list[int], group) -> torch.Tensor:
    """All-to-all of row blocks: block p of `send` (send_counts[p] rows) goes to rank p."""
    world = dist.get_world_size(group)
    out = send.new_empty((sum(recv_counts),) + tuple(send.shape[1:]))
    if dist.get_backend(group) == "nccl":
        dist.all_to_all_single(out, send, recv_counts, send_counts, group=group)
        return out
    # backends without all-to-all (gloo, used by the CPU tests): one broadcast per source rank
    rank = dist.get_rank(group)
    counts = [None] * world
    dist.all_gather_object(counts, send_counts, group=group)
    pos = 0
    for src in range(world):
        total = sum(counts[src])
        buf = send if src == rank else send.new_empty((total,) + tuple(send.shape[1:]))
        dist.broadcast(buf, src=dist.get_global_rank(group, src) if group is not None else src, group=group)
        start = sum(counts[src][:rank])
        n = counts[src][rank]
        out[pos:pos + n] = buf[start:start + n]
        pos += n
    return out


class ExpertParallelMoe:
    def __init__(self, n_expert: int, n_used: int, compute: EpCompute, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if n_expert % self.world:
            raise ValueError(f"{n_expert} experts do not split over {self.world} ranks")
        self.n_expert, self.n_used = n_expert, n_used
        self.per_rank = n_expert // self.world
        self.compute = compute
        self.last_load = None  # rows this rank's experts received in the last forward

    def local_expert_range(self):
        return self.rank * self.per_rank, (self.rank + 1) * self.per_rank

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x: [T, h] on this rank's device -> y [T, h]."""
        T, h = x.shape
        K = self.n_used
        ids, wts = self.compute.route(x)
        flat = ids.reshape(-1).to(torch.int64)
        owner = torch.div(flat, self.per_rank, rounding_mode="floor")
        order = torch.argsort(owner, stable=True)            # pairs grouped by owner, pair order kept inside
        send_counts_t = torch.bincount(owner, minlength=self.world)[: self.world]
        recv_counts_t = torch.empty_like(send_counts_t)
        if dist.get_backend(self.group) == "nccl":
            dist.all_to_all_single(recv_counts_t, send_counts_t, group=self.group)
        else:
            gathered = [torch.empty_like(send_counts_t) for _ in range(self.world)]
            dist.all_gather(gathered, send_counts_t, group=self.group)
            recv_counts_t = torch.stack([g[self.rank] for g in gathered])
        send_counts = send_counts_t.tolist()                 # the one host read of the layer
        recv_counts = recv_counts_t.tolist()
        token_of = torch.div(order, K, rounding_mode="floor")
        send_rows = x.index_select(0, token_of)
        send_ids = (flat.index_select(0, order) - owner.index_select(0, order) * self.per_rank).to(torch.int32)
        recv_rows = _exchange_rows(send_rows, send_counts, recv_counts, self.group)
        recv_ids = _exchange_rows(send_ids, send_counts, recv_counts, self.group)
        self.last_load = int(recv_rows.shape[0])
        out_rows = self.compute.experts(recv_rows, recv_ids) if recv_rows.shape[0] else recv_rows
        back = _exchange_rows(out_rows, recv_counts, send_counts, self.group)   # sorted-pair order again
        per_pair = torch.empty_like(back)
        per_pair.index_copy_(0, order, back)
        # fixed slot order: a sequential sum over the k slots
        y = torch.zeros_like(x)
        pp = per_pair.reshape(T, K, h)
        for s in range(K):
            y.addcmul_(pp[:, s, :], wts[:, s:s + 1])
        return y


def cuda_compute(router_layer, expert_layer) -> EpCompute:
    """EpCompute over two `joshua_b200.moe.Moe` layers: a router-only layer with the global expert count and
    a layer holding this rank's expert banks."""
    k = router_layer.cfg.n_used

    def route(x):
        ids = torch.empty(x.shape[0], k, dtype=torch.int32, device=x.device)
        wts = torch.empty(x.shape[0], k, dtype=torch.float32, device=x.device)
        router_layer.route_dev(x.contiguous(), ids, wts)
        return ids, wts

    def experts(rows, local_ids):
        rows = rows.contiguous()
        out = torch.empty_like(rows)
        expert_layer.experts_dev(rows, local_ids.contiguous(), out)
        return out

    return EpCompute(route, experts)
