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


def _all_to_all_equal(out: torch.Tensor, inp: torch.Tensor, group) -> None:
    """Equal-split all-to-all: block p of `inp` goes to rank p."""
    if dist.get_backend(group) == "nccl":
        dist.all_to_all_single(out, inp, group=group)
        return
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    gathered = [torch.empty_like(inp) for _ in range(world)]
    dist.all_gather(gathered, inp, group=group)
    n = inp.shape[0] // world
    for src in range(world):
        out[src * n:(src + 1) * n] = gathered[src][rank * n:(rank + 1) * n]


def _forward_fixed(self, x: torch.Tensor) -> torch.Tensor:
    """The same layer without any host read: every rank sends every peer a block of fixed capacity
    T * k rows (unused rows carry an out-of-range expert id and come back as zeros), so all sizes are known
    up front and the layer can be captured in a CUDA graph.  Meant for decode-sized batches."""
    T, h = x.shape
    K, W = self.n_used, self.world
    cap = T * K
    ids, wts = self.compute.route(x)
    flat = ids.reshape(-1).to(torch.int64)
    owner = torch.div(flat, self.per_rank, rounding_mode="floor")
    order = torch.argsort(owner, stable=True)
    counts = torch.bincount(owner, minlength=W)[:W]
    starts = torch.cumsum(counts, 0) - counts
    owner_sorted = owner.index_select(0, order)
    slot_sorted = owner_sorted * cap + (torch.arange(cap, device=x.device) - starts.index_select(0, owner_sorted))
    slot = torch.empty_like(slot_sorted)
    slot.index_copy_(0, order, slot_sorted)                      # slot of pair p in the send buffer
    send_rows = x.new_zeros((W * cap, h))
    send_ids = torch.full((W * cap,), self.per_rank, dtype=torch.int32, device=x.device)  # out of range = unused
    token_of = torch.div(torch.arange(cap, device=x.device), K, rounding_mode="floor")
    send_rows.index_copy_(0, slot, x.index_select(0, token_of))
    send_ids.index_copy_(0, slot, (flat - owner * self.per_rank).to(torch.int32))
    recv_rows = torch.empty_like(send_rows)
    recv_ids = torch.empty_like(send_ids)
    _all_to_all_equal(recv_rows, send_rows, self.group)
    _all_to_all_equal(recv_ids, send_ids, self.group)
    out_rows = self.compute.experts(recv_rows, recv_ids)
    back = torch.empty_like(out_rows)
    _all_to_all_equal(back, out_rows, self.group)
    per_pair = back.index_select(0, slot).reshape(T, K, h)
    y = torch.zeros_like(x)
    for s in range(K):
        y.addcmul_(per_pair[:, s, :], wts[:, s:s + 1])
    return y


ExpertParallelMoe.forward_fixed = _forward_fixed


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


class PeerExchange:
    """The exchange of `ExpertParallelMoe` done by the library's own kernels: rows are stored straight into
    the owning rank's memory over NVLink (CUDA IPC mappings) and polled for with bounded waits, with no
    collective call and no host read, so a whole decode step can be one CUDA graph.  One object serves every
    layer of a model.  `torch.distributed` is used once, to hand the window handles round."""

    def __init__(self, ctx, n_expert: int, n_used: int, hidden: int, max_tokens: int, group=None):
        import ctypes

        from . import _lib

        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.ctx = ctx
        self.hidden, self.max_tokens = hidden, max_tokens
        self.rows = self.world * max_tokens * n_used      # rows the local expert layer must be reserved for
        self._h = ctypes.c_void_p()
        _lib.check(_lib.lib().jq_ep_create(ctx._h, self.rank, self.world, n_expert, n_used, hidden, max_tokens,
                                           ctypes.byref(self._h)))
        if self.world > 1:
            mine = (ctypes.c_uint8 * 64)()
            _lib.check(_lib.lib().jq_ep_export(self._h, mine))
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(mine), group=group)
            blob = (ctypes.c_uint8 * (64 * self.world)).from_buffer_copy(b"".join(handles))
            _lib.check(_lib.lib().jq_ep_connect(self._h, blob))
            dist.barrier(group=group)                      # nobody stores into a window that is not mapped yet

    def forward_dev(self, router_layer, expert_layer, x, y, residual=None, stream=None, norm_w=None, eps=0.0,
                    forced_ids=None) -> None:
        """y = (residual +) layer(x), or layer(rmsnorm(x; norm_w, eps)) with `norm_w`; `residual` may be `y`.
        More tokens than the window was sized for go through it in slices of `max_tokens` (every rank must
        then pass the same number of tokens, so that all ranks make the same number of exchanges)."""
        from . import _lib

        T = x.numel() // self.hidden
        s = torch.cuda.current_stream(x.device).cuda_stream if stream is None else stream
        x2, y2 = x.reshape(T, self.hidden), y.reshape(T, self.hidden)
        r2 = residual.reshape(T, self.hidden) if residual is not None else None
        for t0 in range(0, T, self.max_tokens):
            t1 = min(T, t0 + self.max_tokens)
            _lib.check(_lib.lib().jq_ep_forward_norm_dev(
                self._h, router_layer._h, expert_layer._h, x2[t0:t1].data_ptr(), t1 - t0,
                norm_w.data_ptr() if norm_w is not None else None, eps,
                forced_ids[t0:t1].data_ptr() if forced_ids is not None else None,
                r2[t0:t1].data_ptr() if r2 is not None else None, y2[t0:t1].data_ptr(), s))

    def rows_served(self) -> int:
        """Rows this rank's experts were sent in the last exchange (synchronises the device)."""
        import ctypes

        from . import _lib

        n = ctypes.c_uint32()
        _lib.check(_lib.lib().jq_ep_rows_served(self._h, ctypes.byref(n)))
        return int(n.value)

    def close(self) -> None:
        from . import _lib

        if self._h:
            _lib.lib().jq_ep_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
