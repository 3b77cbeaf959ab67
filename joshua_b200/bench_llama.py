"""The `llama8b` benchmark workload: batch-1 decode of a Llama-8B-shaped model with every linear in Q4_K.

The model is `joshua_b200.llama.LlamaDecoder`: random-init, 32 layers, hidden 4096, 32 query / 8 KV heads of
128, SwiGLU FFN 14336, vocabulary 128256, all linears and the embedding as raw Q4_K blocks.  The KV cache is
first filled by feeding token id 42 for `--prefill` positions (the reference's own benchmark feeds a repeated
token, examples/bench_qwen3moe.rs:148-162) in one prefill pass, which is timed and reported as `prefill`; then one timed step = one greedily decoded
token: embedding row, 32 x {RMS norm, fused QKV matmul, RoPE + cache append, attention over the cache, output
projection, residual + RMS norm, gate/up matmul with SwiGLU, down matmul}, final norm, output head, arg-max.
Everything runs on the device; the step is one CUDA graph.  4.22 GB of weights are read per token.

With --gpus N > 1 every rank holds a full replica (dense weights are replicated by design; only MoE expert
banks shard) and decodes its own sequence: weak scaling with no data-path collective, whole-job tokens/s =
N x per-rank.
"""
from __future__ import annotations

import json
import os
import time

import numpy as np

from . import synth
from .llama import LlamaConfig, LlamaDecoder


def run(args, emit=True):
    """Measures the workload; prints the JSON line on rank 0 (emit) and returns it (None on other ranks)."""
    import torch
    import torch.distributed as dist

    from bench import ClockSampler, cpu_llama_sample, measured_peaks

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()

    warmup = max(3, args.warmup)
    cfg = LlamaConfig()
    batch = args.batch
    max_ctx = args.prefill + 2 * (warmup + args.steps) + 16   # device-timed steps, then the host-buffer steps
    model = LlamaDecoder(cfg, dev, batch=batch, max_ctx=max_ctx, seed=rank)
    stream = torch.cuda.Stream()

    def capture(fn):
        with torch.cuda.stream(stream):
            fn()
            fn()
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                fn()
        return g

    step_graph = capture(model.step)
    mm_graph = capture(model.matmuls_only)
    if batch > 1:   # several sequences: fill the cache step by step (prefill handles one sequence)
        with torch.cuda.stream(stream):
            model.reset(42)
            for _ in range(args.prefill):  # the same token at every position
                step_graph.replay()
                model.force_token(42)
            stream.synchronize()

    def timed(graph, steps, warm):
        with torch.cuda.stream(stream):
            for _ in range(warm):
                graph.replay()
            stream.synchronize()
            barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(stream)
            for _ in range(steps):
                graph.replay()
            e.record(stream)
            stream.synchronize()
            barrier()
        return s.elapsed_time(e) * 1e-3 / steps

    # prefill: the prompt in one pass (batched linears on the tile GEMM, causal attention), batch 1 only
    prefill_info = None
    if batch == 1 and args.prefill > 0:
        with torch.cuda.stream(stream):
            model.reset(42)
            model.prefill([42] * args.prefill)          # warm-up (allocations, kernel loading)
            times = []
            for _ in range(3):
                model.reset(42)
                stream.synchronize()
                s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s0.record(stream)
                model.prefill([42] * args.prefill)
                e0.record(stream)
                stream.synchronize()
                times.append(s0.elapsed_time(e0) * 1e-3)
            pt = sorted(times)[1]
            prefill_info = {"tokens": args.prefill, "ms": pt * 1e3, "tok_s": args.prefill / pt,
                            "tflops_algorithmic": 2.0 * args.prefill * (model.weight_bytes / 0.5625) / pt / 1e12,
                            "how": "LlamaDecoder.prefill: one pass over the prompt, median of 3 (eager launches)"}
            model.check_flags()
            # the cache now holds the prompt; the timed decode steps continue from it
    with ClockSampler(local) as clocks:
        dt = timed(step_graph, args.steps, warmup)
    assert int(model.bad.item()) == 0 and int(model.pos.max().item()) < max_ctx
    dt_mm = timed(mm_graph, args.steps, warmup)
    if world > 1:
        tmax = torch.tensor([dt], device=dev, dtype=torch.float64)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dt = float(tmax.item())

    # end to end, model level: host token ids in, host logits out, every step (pinned buffers), on every rank
    tok = np.full(batch, 42, np.int32)
    for _ in range(3):
        model.forward_host(tok)
    torch.cuda.synchronize()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        logits_host = model.forward_host(tok)
        tok = logits_host.argmax(axis=1).astype(np.int32)   # the host picks the next token from the logits
    e2e_dt = (time.perf_counter() - t0) / args.steps
    h2d, d2h = 4 * batch * world, 4 * batch * cfg.vocab * world
    if world > 1:
        tmax = torch.tensor([e2e_dt], device=dev, dtype=torch.float64)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        e2e_dt = float(tmax.item())

    if rank == 0:
        # end to end, operator level: every matmul of the token through jq_matmul_t with host buffers (layer 0 and
        # the head timed, x layers)
        ly = model.layers[0]
        c = cfg
        qs = [(ly["wqkv"], c.qkv_rows, c.hidden, c.hidden), (ly["wo"], c.hidden, c.q_heads * c.head_dim, c.hidden),
              (ly["w_gate"], c.ffn, c.hidden, c.hidden), (ly["w_up"], c.ffn, c.hidden, c.hidden),
              (ly["w_down"], c.hidden, c.ffn, c.ffn)]
        x_host = {k: np.random.default_rng(0).standard_normal((batch, k)).astype(np.float32) for k in (c.hidden, c.ffn)}

        def host_layer():
            for q, n, k, inp in qs:
                q.matmul_t((batch, k, n), x_host[inp])

        for _ in range(3):
            host_layer()
        reps = 10
        t0 = time.perf_counter()
        for _ in range(reps):
            host_layer()
        per_layer = (time.perf_counter() - t0) / reps
        model.output.matmul_t((batch, c.hidden, c.vocab), x_host[c.hidden])
        t0 = time.perf_counter()
        for _ in range(reps):
            model.output.matmul_t((batch, c.hidden, c.vocab), x_host[c.hidden])
        per_head = (time.perf_counter() - t0) / reps
        op_dt = per_layer * c.layers + per_head

        peak, which = measured_peaks()
        alg = model.algorithmic_bytes()
        launches = model.matmuls_per_step
        ach = alg / dt_mm / 1e9
        line = {
            "metric": "decode_tok_s", "value": world * batch / dt, "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 codes x int8 activation planes -> int32, f32 scales and glue", "data": "synthetic",
            "config": {"workload": f"llama8b_q4k_decode_b{batch}", "layers": c.layers, "hidden": c.hidden,
                       "q_heads": c.q_heads, "kv_heads": c.kv_heads, "head_dim": c.head_dim, "ffn": c.ffn,
                       "vocab": c.vocab, "batch": batch, "prefill": args.prefill,
                       "step": "full decode step on the device (embedding, norms, RoPE, attention over the KV cache, "
                               "quantized matmuls, greedy arg-max), one CUDA graph; "
                               "five launches per layer",
                       "l2": "4.22 GB of weights per step, far larger than L2", "parallelism": f"replicas x{world}"},
            "e2e": {"value": world * batch / e2e_dt, "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "how": "model-level call with host buffers (LlamaDecoder.forward_host, the shape of the "
                           "reference's ModelWeights::forward): token ids host->device, one decode step, logits "
                           "device->host, the host picks the next token; wall clock over the timed steps",
                    "operator_level_tok_s": batch / op_dt,
                    "operator_level_how": "every linear of the token through jq_matmul_t with host slices (the "
                                          "QuantizedType::matmul_t boundary): layer 0 and the head timed, x layers"},
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                         # an ncu capture of the 28672 x 4096 launch: its dram read + write is
                         # 66.44 MB against 66.08 MB algorithmic, i.e. x 1.005; scaled to the average launch here
                         "traffic": alg / launches * 1.005, "traffic_unit": "bytes per launch (average launch)",
                         "peak_source": which, "kernel": "gemv_mma_kernel<Q4_K>",
                         "launches_per_step": launches, "avg_launch_us": dt_mm / launches * 1e6,
                         "bytes_per_step": alg},
            "gpu_launches": model.launches_per_step * args.steps, "clocks": clocks.summary(),
            "prefill": prefill_info,
        }
        try:
            base = cpu_llama_sample(seconds_budget=12.0)
            line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        except Exception as exc:  # the oracle is test infrastructure; the line stands without it
            line["cpu_baseline"] = {"value": None, "unit": "tok/s", "cores": 0, "kind": "port", "sample": repr(exc)}
        if emit:
            print(json.dumps(line))
    else:
        line = None
    if world > 1:
        dist.destroy_process_group()
    del model
    torch.cuda.empty_cache()
    return line
