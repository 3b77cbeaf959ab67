"""The `qwen3moe` benchmark workload: decode of a Qwen3-MoE-shaped model (48 layers, hidden 2048, 32 query / 4 KV
heads of 128, 128 routed experts top-8 with feed-forward width 768; expert banks Q4_K, attention Q8_0).

One step = one greedily decoded token per sequence, the whole step on the device.  With --gpus N > 1 the expert
banks are split over the ranks (16 / 32 / 64 experts each at N = 8 / 4 / 2), attention and router weights are
replicated, every rank decodes its own `--batch` sequences and the routed activation rows travel by direct
stores into the owning rank's memory over NVLink (`csrc/ep.cu`: fixed-capacity windows, flag handshakes, no
collective call and no host read, so a whole step is one CUDA graph).  Whole-job tokens/s = N x batch / step
time; per-GPU work is fixed as N grows (weak scaling).  The line also carries `strong`: the same model at a
fixed global batch of 16 sequences (16 / N per GPU), and `load`: max / mean rows per rank.
"""
from __future__ import annotations

import json
import os

from . import synth
from .moe_decoder import MoeDecoder, MoeDecoderConfig


def moe_config(cfg, batch: int, world: int) -> dict:
    """The `config` object of the workload; the reference arm prints the same one."""
    return {"workload": f"qwen3moe_decode_b{batch}", "layers": cfg.layers, "hidden": cfg.hidden,
            "n_expert": cfg.n_expert, "n_used": cfg.n_used, "moe_inter": cfg.moe_inter, "experts": "q4_k",
            "attention": "q8_0", "batch_per_gpu": batch, "parallelism": f"ep{world}" if world > 1 else "single",
            "l2": "about 2 GB of weights per step, far larger than L2"}


def measure(args, batch: int, group, sample_load: bool = True, with_e2e: bool = True) -> dict:
    """Builds the model at `batch` sequences per GPU, times `args.steps` decode steps (CUDA events, max over ranks)
    and the host-buffer steps; returns the fields of the JSON line (every rank gets the same timing fields)."""
    import time

    import numpy as np
    import torch
    import torch.distributed as dist

    from bench import ClockSampler

    world = dist.get_world_size(group) if group is not None else 1
    rank = dist.get_rank(group) if group is not None else 0
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    warmup = max(3, args.warmup)
    cfg = MoeDecoderConfig()
    prefill = min(args.prefill, 128)
    prompt = args.prefill if (world == 1 and batch == 1 and with_e2e) else 0   # one timed prefill pass, one GPU only
    max_ctx = max(prefill, prompt) + 3 * (warmup + args.steps) + 24
    # the same seed on every rank: attention, router and head weights are replicas; a rank draws only its own experts
    model = MoeDecoder(cfg, dev, batch=batch, max_ctx=max_ctx, seed=0, group=group)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        model.reset(42)
        # every sequence starts from its own token so that the ranks (and the sequences of a batch) route differently
        model.token.copy_(torch.arange(batch, dtype=torch.int32) + 42 + 1000 * rank)
        model.step()
        model.step()
        stream.synchronize()
        barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            model.step()
        stream.synchronize()
        for _ in range(prefill + warmup):
            graph.replay()
        stream.synchronize()
        barrier()
        with ClockSampler(local) as clocks:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(stream)
            for _ in range(args.steps):
                graph.replay()
            e.record(stream)
            stream.synchronize()
        barrier()
        dt = max_over_ranks(s.elapsed_time(e) * 1e-3 / args.steps)
        # the quantized matmuls of the step alone (the dominant kernel, gemv_mma_kernel: dense Q8_0 linears, grouped
        # Q4_K experts over the routing the last step left, head), one CUDA graph, CUDA events
        mm_dt = None
        if with_e2e:
            mm_graph = torch.cuda.CUDAGraph()
            model.matmuls_only(stream.cuda_stream)
            stream.synchronize()
            with torch.cuda.graph(mm_graph, stream=stream):
                model.matmuls_only(stream.cuda_stream)
            for _ in range(3):
                mm_graph.replay()
            stream.synchronize()
            s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s2.record(stream)
            for _ in range(args.steps):
                mm_graph.replay()
            e2.record(stream)
            stream.synchronize()
            mm_dt = max_over_ranks(s2.elapsed_time(e2) * 1e-3 / args.steps)
        # load balance: rows each rank's experts were sent in the last layer of a step, sampled over a few steps
        load = None
        if world > 1 and sample_load:
            served = []
            for _ in range(8):
                graph.replay()
                stream.synchronize()
                mine = torch.tensor([float(model.exchange.rows_served())], device=dev, dtype=torch.float64)
                rows = [torch.zeros_like(mine) for _ in range(world)]
                dist.all_gather(rows, mine)
                served.append([float(r.item()) for r in rows])
            a = np.array(served)
            load = {"max_over_mean_rows_per_rank": float((a.max(axis=1) / np.maximum(a.mean(axis=1), 1e-9)).mean()),
                    "rows_per_rank_mean": float(a.mean()), "sampled": "last layer of 8 steps"}
    model.check_flags()
    out = {"dt": dt, "mm_dt": mm_dt, "clocks": clocks.summary(), "load": load, "cfg": cfg, "warmup": warmup,
           "launches_per_step": model.launches_per_step, "weight_bytes": model.weight_bytes}
    if prompt > 0:
        # the prompt in one pass (`forward(input [1, seq_len], 0)`): batched linears and the experts' buckets on the
        # tile GEMM, causal attention; the reference's bench feeds a repeated token (examples/bench_qwen3moe.rs:148-162)
        with torch.cuda.stream(stream):
            ids = ((np.arange(prompt) * 7919) % 50000 + 42).astype(np.int32)   # distinct tokens: the experts all see rows
            model.reset(42)
            model.prefill(ids)
            times = []
            for _ in range(3):
                model.reset(42)
                stream.synchronize()
                s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s0.record(stream)
                model.prefill(ids)
                e0.record(stream)
                stream.synchronize()
                times.append(s0.elapsed_time(e0) * 1e-3)
            pt = sorted(times)[1]
        model.check_flags()
        out["prefill"] = {"tokens": prompt, "ms": pt * 1e3, "tok_s": prompt / pt,
                          "how": "MoeDecoder.prefill: one pass over the prompt, median of 3 (eager launches)"}
    if with_e2e:
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
        out["e2e_dt"] = max_over_ranks((time.perf_counter() - t0) / args.steps)
        model.check_flags()
    if getattr(model, "exchange", None) is not None:
        barrier()
        model.exchange.close()
    del model
    torch.cuda.empty_cache()
    return out


def run(args, extra=None):
    """Prints the workload's JSON line (rank 0).  `extra(line)` may add objects to it before it is printed."""
    import torch
    import torch.distributed as dist

    from bench import cpu_moe_sample, measured_peaks

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
    batch = args.batch
    m = measure(args, batch, group)
    cfg, dt, e2e_dt, mm_dt = m["cfg"], m["dt"], m["e2e_dt"], m["mm_dt"]
    # strong scaling at a fixed global batch of 16 sequences (the configuration's "batch 16"): 16 / N per GPU
    strong = None
    if getattr(args, "strong", True) and 16 % world == 0:
        sm = measure(args, 16 // world, group, sample_load=True, with_e2e=False)
        strong = {"global_batch": 16, "batch_per_gpu": 16 // world, "value": 16 / sm["dt"], "unit": "tok/s",
                  "ms_per_step": sm["dt"] * 1e3, "scaling": "strong", "load": sm["load"]}
    if rank == 0:
        peak, which = measured_peaks()
        # bytes one rank's step must read: attention weights + head once, expert banks once per distinct expert
        # touched (at most batch * k per layer, each 3 matrices)
        per_expert = 2 * synth.tensor_bytes(synth.Q4_K, cfg.moe_inter, cfg.hidden) + \
            synth.tensor_bytes(synth.Q4_K, cfg.hidden, cfg.moe_inter)
        touched = min(cfg.n_expert, batch * cfg.n_used)
        alg = m["weight_bytes"] + cfg.layers * touched * per_expert
        line = {
            "metric": "decode_tok_s", "value": world * batch / dt, "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": m["warmup"], "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 codes x int8 activation planes -> int32, f32 scales and glue", "data": "synthetic",
            "config": moe_config(cfg, batch, world),
            "roofline": {"bound": "hbm", "achieved": alg / mm_dt / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": alg / mm_dt / 1e9 / peak, "traffic": None, "peak_source": which,
                         "kernel": "gemv_mma_kernel: the step's quantized matmuls alone (per layer the Q8_0 QKV and output "
                                   "projections and the grouped Q4_K gate/up and down products of the routed experts, "
                                   "then the head), one CUDA graph, CUDA events",
                         "bytes_per_step": alg, "ms": mm_dt * 1e3,
                         "step_frac": alg / dt / 1e9 / peak,
                         "note": "bytes = the weight bytes one rank must read per step: attention + head once, 3 matrices "
                                 "per distinct expert touched; step_frac = the same bytes over the whole step (all "
                                 "kernels, and at N > 1 the exchange)"},
            "e2e": {"value": world * batch / e2e_dt, "unit": "tok/s", "h2d_bytes_per_step": 4 * batch * world,
                    "d2h_bytes_per_step": 4 * batch * cfg.vocab * world,
                    "how": "model-level call with host buffers on every rank (forward_host): token ids host->device, "
                           "one decode step, logits device->host, the host picks the next token; wall clock, max "
                           "over ranks"},
            "gpu_launches": m["launches_per_step"] * args.steps, "clocks": m["clocks"],
            "exchange": None if world == 1 else "peer-memory stores over NVLink (csrc/ep.cu), one CUDA graph per step",
            "load": m["load"], "strong": strong, "prefill": m.get("prefill"),
        }
        if world == 1:
            try:
                base = cpu_moe_sample(cfg, seconds_budget=10.0)
                line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
            except Exception as exc:  # the oracle is test infrastructure; the line stands without it
                line["cpu_baseline"] = {"value": None, "unit": "tok/s", "cores": 0, "kind": "port", "sample": repr(exc)}
        if extra is not None:
            extra(line)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
