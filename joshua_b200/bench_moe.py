"""The `qwen3moe` benchmark workload: decode of a Qwen3-MoE-shaped model (48 layers, hidden 2048, 32 query / 4 KV
heads of 128, 128 routed experts top-8 with feed-forward width 768; expert banks Q4_K, attention Q8_0).

One step = one greedily decoded token per sequence, the whole step on the device.  With --gpus N > 1 the expert
banks are split over the ranks (16 / 32 / 64 experts each at N = 8 / 4 / 2), attention and router weights are
replicated, every rank decodes its own `--batch` sequences and the routed activation rows travel by NCCL
all-to-all (fixed-capacity exchange, no host read, so the step is one CUDA graph when the collective can be
captured).  Whole-job tokens/s = N x batch / step time; per-GPU work is fixed as N grows (weak scaling).
"""
from __future__ import annotations

import json
import os

from . import synth
from .moe_decoder import MoeDecoder, MoeDecoderConfig


def run(args):
    import torch
    import torch.distributed as dist

    import time

    import numpy as np

    from bench import ClockSampler, cpu_moe_sample, measured_peaks

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

    def barrier():
        if world > 1:
            dist.barrier()

    warmup = max(3, args.warmup)
    cfg = MoeDecoderConfig()
    batch = args.batch
    prefill = min(args.prefill, 128)
    max_ctx = prefill + 3 * (warmup + args.steps) + 24
    model = MoeDecoder(cfg, dev, batch=batch, max_ctx=max_ctx, seed=rank, group=group)
    stream = torch.cuda.Stream()
    graph = None
    with torch.cuda.stream(stream):
        model.reset(42)
        model.step()
        model.step()
        stream.synchronize()
        barrier()
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                model.step()
            graph = g
        except Exception as exc:  # collectives that cannot be captured: run the step eagerly
            if rank == 0:
                print(f"# graph capture unavailable ({type(exc).__name__}); timing eager steps", flush=True)
            graph = None
        stream.synchronize()

    def one():
        if graph is not None:
            graph.replay()
        else:
            model.step()

    with torch.cuda.stream(stream):
        model.reset(42)
        for _ in range(prefill):
            one()
            model.force_token(42)
        for _ in range(warmup):
            one()
        stream.synchronize()
        barrier()
        with ClockSampler(local) as clocks:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(stream)
            for _ in range(args.steps):
                one()
            e.record(stream)
            stream.synchronize()
        barrier()
    dt = s.elapsed_time(e) * 1e-3 / args.steps
    assert int(model.pos.max().item()) < max_ctx
    if world > 1:
        tmax = torch.tensor([dt], device=dev, dtype=torch.float64)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dt = float(tmax.item())
    # end to end, model level: host token ids in, host logits out, every step (every rank does its own copies)
    tok = np.full(batch, 42, np.int32)
    for _ in range(3):
        model.forward_host(tok)
    torch.cuda.synchronize()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        logits_host = model.forward_host(tok)
        tok = logits_host.argmax(axis=1).astype(np.int32)
    e2e_dt = (time.perf_counter() - t0) / args.steps
    if world > 1:
        tmax = torch.tensor([e2e_dt], device=dev, dtype=torch.float64)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        e2e_dt = float(tmax.item())
    assert int(model.pos.max().item()) < max_ctx
    if rank == 0:
        peak, which = measured_peaks()
        # bytes one rank's step must read: attention weights + head once, expert banks once per distinct expert
        # touched (at most batch * k per layer, each 3 matrices)
        per_expert = 2 * synth.tensor_bytes(synth.Q4_K, cfg.moe_inter, cfg.hidden) + \
            synth.tensor_bytes(synth.Q4_K, cfg.hidden, cfg.moe_inter)
        touched = min(cfg.n_expert, batch * cfg.n_used)
        alg = model.weight_bytes + cfg.layers * touched * per_expert
        line = {
            "metric": "decode_tok_s", "value": world * batch / dt, "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 codes x int8 activation planes -> int32, f32 scales and glue", "data": "synthetic",
            "config": {"workload": f"qwen3moe_decode_b{batch}", "layers": cfg.layers, "hidden": cfg.hidden,
                       "n_expert": cfg.n_expert, "n_used": cfg.n_used, "moe_inter": cfg.moe_inter,
                       "experts": "q4_k", "attention": "q8_0", "batch_per_gpu": batch, "prefill": prefill,
                       "parallelism": f"ep{world}" if world > 1 else "single", "cuda_graph": graph is not None,
                       "l2": "about 2 GB of weights per step, far larger than L2"},
            "roofline": {"bound": "hbm", "achieved": alg / dt / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": alg / dt / 1e9 / peak, "traffic": None, "peak_source": which,
                         "note": "whole step (all kernels) over the weight bytes one rank must read, upper bound "
                                 "on distinct experts"},
            "e2e": {"value": world * batch / e2e_dt, "unit": "tok/s", "h2d_bytes_per_step": 4 * batch * world,
                    "d2h_bytes_per_step": 4 * batch * cfg.vocab * world,
                    "how": "model-level call with host buffers on every rank (forward_host): token ids host->device, "
                           "one decode step, logits device->host, the host picks the next token; wall clock, max "
                           "over ranks"},
            "gpu_launches": model.launches_per_step * args.steps, "clocks": clocks.summary(),
        }
        if world == 1:
            try:
                base = cpu_moe_sample(cfg, seconds_budget=10.0)
                line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
            except Exception as exc:  # the oracle is test infrastructure; the line stands without it
                line["cpu_baseline"] = {"value": None, "unit": "tok/s", "cores": 0, "kind": "port", "sample": repr(exc)}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
