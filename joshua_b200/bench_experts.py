"""The `mxfp4_experts` benchmark workload: one routed-expert layer of a Kimi-class shape - 384 experts top-8, hidden
7168, expert width 2048, MXFP4 banks (8.98 GB) - swept over 1 / 16 / 256 / 4096 tokens with Zipf(1.1) expert
popularity, on 1 / 2 / 4 / 8 GPUs.

Inputs are synthetic: raw MXFP4 blocks with uniform codes and scale exponents in [118, 130], activations drawn
N(0, 1) in bf16 and widened to f32 (the reference has no bf16 entry, src/mxfp4.rs:242-258 is f16 only), and
expert ids sampled per token without replacement (Gumbel top-k) from p(e) ~ 1 / rank(e)^1.1, where the
popularity rank of an expert is a seeded permutation of its index - so that a contiguous split of the experts
over the ranks does not put all popular experts on one GPU by construction.  The ids enter the layer as forced
ids (the mechanism of hash-routed layers, src/quantized_deepseek4.rs:1375-1398); routing weights still come from
the gate.

With --gpus N the banks are split contiguously (48 experts per rank at N = 8), every rank holds `tokens / N`
of the tokens (at least one) and rows travel through the peer-memory exchange of `csrc/ep.cu`, in slices of up
to 2048 tokens per rank.  Reported per token count: tokens/s, algorithmic TFLOP/s (2 * tokens * 8 * 3 * 7168 * 2048),
the GB/s of distinct experts' bytes read (the roofline at 1 and 16 tokens), and max / mean rows per rank.
"""
from __future__ import annotations

import json
import os

import numpy as np

from . import synth
from .moe import GATE_SOFTMAX, OOB_SKIP, Moe, MoeConfig
from .qtensor import QTensor, default_context

E, K, H, INTER = 384, 8, 7168, 2048


def zipf_ids(tokens: int, rng: np.random.Generator, perm: np.ndarray, s: float = 1.1) -> np.ndarray:
    """[tokens, K] distinct expert ids per token, popularity p(e) ~ 1 / (perm[e] + 1)^s."""
    logp = -s * np.log(perm.astype(np.float64) + 1.0)
    g = rng.gumbel(size=(tokens, E))
    return np.argsort(-(logp[None, :] + g), axis=1)[:, :K].astype(np.uint32)


def run(args):
    import torch
    import torch.distributed as dist

    from bench import ClockSampler, measured_peaks

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    group = None
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    ctx = default_context(local)
    t = synth.MXFP4
    per = E // world
    banks, keep = [], []
    for i, (rows, cols) in enumerate([(INTER, H), (INTER, H), (H, INTER)]):
        nbytes = synth.tensor_bytes(t, per * rows, cols)
        raw = torch.cat([synth.random_weight_torch(t, per * rows, cols, 1000 * (31 + i) + rank, dev),
                         torch.zeros(16, dtype=torch.uint8, device=dev)])
        keep.append(raw)
        banks.append(QTensor.from_device(t, raw[:nbytes], ctx))
    router = (np.random.default_rng(0).standard_normal((E, H)) * 0.02).astype(np.float32)
    token_counts = [int(v) for v in str(args.tokens).split(",")]
    if world == 1:
        layer = Moe(MoeConfig(gating=GATE_SOFTMAX, n_expert=E, n_used=K, hidden=H, inter=INTER, norm=True), router,
                    *banks, ctx=ctx)
        exchange = None
    else:
        from .ep import PeerExchange

        rl = Moe(MoeConfig(gating=GATE_SOFTMAX, n_expert=E, n_used=K, hidden=H, inter=INTER, norm=True), router, None,
                 None, None, ctx=ctx)
        el = Moe(MoeConfig(gating=GATE_SOFTMAX, n_expert=per, n_used=1, hidden=H, inter=INTER, oob_policy=OOB_SKIP),
                 np.zeros((per, H), np.float32), *banks, ctx=ctx)
        exchange = None
    perm = np.random.default_rng(7).permutation(E)
    per_expert_bytes = 3 * synth.tensor_bytes(t, INTER, H)
    peak, which = measured_peaks()
    sweep = []
    clocks_all = None
    for T in token_counts:
        Tl = max(1, T // world)                                      # tokens this rank holds
        Tg = Tl * world
        sets = 4
        rng = np.random.default_rng(100 + T)
        ids_all = [zipf_ids(Tg, rng, perm) for _ in range(sets)]     # every rank draws the same global ids
        xs = [torch.randn(Tl, H, device=dev, dtype=torch.bfloat16).float() for _ in range(sets)]
        ids = [torch.from_numpy(a[rank * Tl:(rank + 1) * Tl].copy()).to(dev) for a in ids_all]
        y = torch.empty(Tl, H, device=dev)
        if world == 1:
            layer.reserve(Tl, Tl * K)
        else:
            # the exchange is sized for this token count (its fixed-capacity blocks cost time in proportion)
            if exchange is not None:
                dist.barrier()
                exchange.close()
            cap = min(2048, Tl)                                      # tokens per rank and exchange
            exchange = PeerExchange(ctx, E, K, H, cap, group=group)
            rl.reserve(cap, 0)
            el.reserve(cap * K * world, cap * K * world)
        it = [0]

        def step():
            i = it[0] % sets
            if world == 1:
                layer.forward_dev(xs[i], y, forced_ids=ids[i])
            else:
                exchange.forward_dev(rl, el, xs[i], y, forced_ids=ids[i])
            it[0] += 1

        steps = max(2, min(args.steps, 8 if T >= 4096 else args.steps))
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        with ClockSampler(local) as clocks:
            s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            for _ in range(steps):
                step()
            e0.record()
            torch.cuda.synchronize()
        dt = s0.elapsed_time(e0) * 1e-3 / steps
        if world > 1:
            tm = torch.tensor([dt], device=dev, dtype=torch.float64)
            dist.all_reduce(tm, op=dist.ReduceOp.MAX)
            dt = float(tm.item())
        clocks_all = clocks.summary()
        # figures from the ids themselves: distinct experts (bytes that must be read) and rows per owning rank
        distinct = float(np.mean([len(np.unique(a)) for a in ids_all]))
        rows = np.array([[np.count_nonzero(a // per == r) for r in range(world)] for a in ids_all], dtype=np.float64)
        flops = 2.0 * Tg * K * 3 * H * INTER
        sweep.append({
            "tokens": Tg, "tokens_per_gpu": Tl, "ms": dt * 1e3, "tok_s": Tg / dt, "tflops_algorithmic": flops / dt / 1e12,
            "distinct_experts": distinct, "expert_gbs": distinct * per_expert_bytes / dt / 1e9,
            "frac_of_hbm_all_gpus": distinct * per_expert_bytes / dt / 1e9 / (peak * world),
            "max_over_mean_rows_per_rank": float((rows.max(axis=1) / np.maximum(rows.mean(axis=1), 1e-9)).mean()),
        })
    if world == 1:
        layer.status()
    if rank == 0:
        big = sweep[-1]
        line = {
            "metric": "moe_layer_tok_s", "value": big["tok_s"], "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": 3, "ms_per_step": big["ms"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8 codes x int8 activation planes -> int32 (decode sizes); tf32 x3 on tcgen05 (bucketed sizes)",
            "data": "synthetic",
            "config": {"workload": "mxfp4_experts", "n_expert": E, "n_used": K, "hidden": H, "inter": INTER,
                       "type": "mxfp4", "routing": "Zipf(1.1) popularity over a seeded permutation of the experts, "
                       "8 distinct experts per token", "activations": "bf16 N(0,1) widened to f32",
                       "parallelism": f"ep{world}" if world > 1 else "single",
                       "l2": "8.98 GB of banks; token sets and ids change every call"},
            "sweep": sweep,
            "roofline": {"bound": "hbm", "achieved": sweep[0]["expert_gbs"], "peak": peak * world, "unit": "GB/s",
                         "frac": sweep[0]["frac_of_hbm_all_gpus"], "traffic": None, "peak_source": which,
                         "note": f"distinct experts' bytes at {sweep[0]['tokens']} token(s); larger counts are "
                                 "compute-bound, see sweep[].tflops_algorithmic"},
            "gpu_launches": None, "clocks": clocks_all,
        }
        print(json.dumps(line))
    if exchange is not None:
        dist.barrier()
        exchange.close()
    if world > 1:
        dist.destroy_process_group()
