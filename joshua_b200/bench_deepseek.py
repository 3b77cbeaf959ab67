"""The `deepseek_v3` benchmark workload: decode of a DeepSeek-V3-shaped stack of 8 MoE layers with multi-head latent
attention (hidden 7168, 128 heads, q_lora 1536, kv_lora 512, rope 64; nope and value head sizes 128 / 128 - the
configuration does not give them, these are V3's), 256 routed experts top-8 (8 groups, 4 kept, sigmoid scores with
selection bias, weights renormalised and scaled by 2.5) plus one shared expert of width 2048; routed banks
IQ2_XXS, everything else Q8_0; plain rotary embedding (YaRN factor 1).  Random-init: the reference's own
`deepseek2` loader cannot read IQ2_XXS tensors (src/gguf_ext.rs:238-276), so this model is a composition of its
MLA / routing code with its IQ2_XXS kernels, validated against the CPU model of tests/cpu_model.py.

One step = one greedily decoded token per sequence, the whole step on the device, one CUDA graph.  With --gpus N
the routed banks are split over the ranks (peer-memory exchange); attention, router, shared expert and head are
replicated and every rank decodes its own `--batch` sequences.
"""
from __future__ import annotations

import json
import os

from .deepseek import DeepseekConfig, DeepseekDecoder


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
    warmup, batch = max(3, args.warmup), args.batch
    prefill = min(args.prefill, 128)
    cfg = DeepseekConfig()
    model = DeepseekDecoder(cfg, dev, batch=batch, max_ctx=prefill + warmup + args.steps + 16, seed=0, group=group)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        model.reset(42)
        model.token.copy_(torch.arange(batch, dtype=torch.int32) + 42 + 1000 * rank)
        model.step()
        model.step()
        stream.synchronize()
        if world > 1:
            dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            model.step()
        for _ in range(prefill + warmup):
            graph.replay()
        stream.synchronize()
        if world > 1:
            dist.barrier()
        with ClockSampler(local) as clocks:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(stream)
            for _ in range(args.steps):
                graph.replay()
            e.record(stream)
            stream.synchronize()
    dt = s.elapsed_time(e) * 1e-3 / args.steps
    if world > 1:
        t = torch.tensor([dt], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
    model.check_flags()
    if rank == 0:
        peak, which = measured_peaks()
        alg = model.bytes_per_token() if batch == 1 else None
        line = {
            "metric": "decode_tok_s", "value": world * batch / dt, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 codes x int8 activation planes -> int32, f32 scales and glue", "data": "synthetic",
            "config": {"workload": f"deepseek_v3_decode_b{batch}", "layers": cfg.layers, "hidden": cfg.hidden,
                       "n_head": cfg.n_head, "q_lora": cfg.q_lora, "kv_lora": cfg.kv_lora, "qk_nope": cfg.qk_nope,
                       "qk_rope": cfg.qk_rope, "v_dim": cfg.v_dim, "n_expert": cfg.n_expert, "n_used": cfg.n_used,
                       "shared_experts": 1, "moe_inter": cfg.moe_inter, "experts": "iq2_xxs", "rest": "q8_0",
                       "batch_per_gpu": batch, "context": prefill,
                       "parallelism": f"ep{world}" if world > 1 else "single"},
            "roofline": None if alg is None else {
                "bound": "hbm", "achieved": alg / dt / 1e9, "peak": peak, "unit": "GB/s", "frac": alg / dt / 1e9 / peak,
                "traffic": None, "peak_source": which,
                "note": "whole step over the weight bytes one rank reads (dense matrices, head, routed experts "
                        "touched); the per-head K / V cache read (164 KB per position and layer) is not counted",
                "bytes_per_step": alg},
            "gpu_launches": model.launches_per_step * args.steps, "clocks": clocks.summary(),
        }
        print(json.dumps(line))
    if getattr(model, "exchange", None) is not None:
        dist.barrier()
        model.exchange.close()
    if world > 1:
        dist.destroy_process_group()
