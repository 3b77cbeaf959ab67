"""Benchmark of the quantized-matmul path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workloads
  (default) the decode step of the Qwen3-MoE-shaped model at one sequence per GPU - the configuration whose expert
           banks shard: with --gpus N > 1 (under torchrun) the experts are split over the ranks and activation
           rows are exchanged through peer memory over NVLink (csrc/ep.cu).  The line carries `strong` (fixed
           global batch 16) and `load` (max / mean rows per rank); at N = 1 also `dense`, the full line of the
           llama8b workload (the configuration the decode metric is quoted on for dense models), and `kernels`,
           the five block formats' 4096 x 4096 single-matmul GB/s.
  qwen3moe the MoE line alone (--batch sequences per GPU).
  llama8b  decode of a Llama-8B-shaped model, every linear Q4_K, batch 1 (--batch up to 8): the KV cache is
           filled with --prefill positions, then one step = one greedily decoded token, the whole step on the
           device (4.22 GB of raw Q4_K blocks read once per token).  With --gpus N: N replicas, no collective.
  moe_layer one routed-expert layer (--type, --experts, --used, --k hidden, --n expert width, --m tokens):
           the grouped expert matmuls at a given token count.
  deepseek_v3  decode of a DeepSeek-V3-shaped stack: 8 layers of multi-head latent attention + 256 IQ2_XXS experts
           top-8 with a shared expert, the rest Q8_0 (--batch sequences per GPU; experts over --gpus N ranks).
  mxfp4_experts  one routed-expert layer of 384 MXFP4 experts top-8 (hidden 7168, width 2048) swept over
           1 / 16 / 256 / 4096 tokens with Zipf(1.1) expert popularity; with --gpus N the banks are split over the
           ranks and rows cross through the peer-memory exchange (joshua_b200/bench_experts.py).
  gemv     one quantized matmul shape, rotated over a working set larger than L2
           (--type, --n, --k, --m, --rotate-gb): the kernel-level roofline probe
           and the command used for ncu captures.

One JSON line is printed by rank 0.  `value` is tokens/s with inputs resident
in HBM; `e2e` is the same metric through the host-buffer C ABI (`jq_matmul_t`,
host->device and device->host copies inside the timed region); `roofline` is the
dominant kernel's algorithmic bytes over its CUDA-event time against the
measured HBM copy bandwidth; `cpu_baseline` is the CPU oracle (a C++/AVX2
restatement of the reference's kernels) timed on this host's cores on a bounded
sample of the same workload.  `--impl reference` times that CPU path alone.
All data are synthetic (seeded random raw blocks, N(0,1) activations).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402

from joshua_b200 import synth  # noqa: E402

FALLBACK_HBM_GBS = 6650.0
TYPE_BY_NAME = {v: k for k, v in synth.NAMES.items()}

# Llama-8B-class shape of the benchmark configuration
LLAMA = dict(layers=32, hidden=4096, q_heads=32, kv_heads=8, head_dim=128, ffn=14336, vocab=128256)


def llama_linears():
    """(name, n, k) of the quantized linears one decoded token passes through, in order."""
    c = LLAMA
    h, kv = c["hidden"], c["kv_heads"] * c["head_dim"]
    per_layer = [("wq", h, h), ("wk", kv, h), ("wv", kv, h), ("wo", h, h),
                 ("w_gate", c["ffn"], h), ("w_up", c["ffn"], h), ("w_down", h, c["ffn"])]
    out = []
    for layer in range(c["layers"]):
        out += [(f"l{layer}.{nm}", n, k) for nm, n, k in per_layer]
    out.append(("output", c["vocab"], h))
    return out


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i", str(self.index),
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) == 6:
                self.rows.append(parts)

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = sorted(float(r[0]) for r in self.rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(self.rows[0][1]), "reasons": reasons,
                "samples": len(self.rows)}


# ───────────────────────────── CPU baseline ───────────────────────────────

def cpu_llama_sample(seconds_budget: float = 15.0):
    """Times the oracle on layer-0's seven linears + nothing else, scaled to a token.

    The sample is a fixed fraction of the token's weight bytes; tokens/s is
    extrapolated by bytes (every linear is the same Q4_K kernel at m = 1).
    """
    import oracle

    c = LLAMA
    h, kv = c["hidden"], c["kv_heads"] * c["head_dim"]
    shapes = [(h, h), (kv, h), (kv, h), (h, h), (c["ffn"], h), (c["ffn"], h), (h, c["ffn"])]
    weights = [synth.random_weight(synth.Q4_K, n, k, seed=i) for i, (n, k) in enumerate(shapes)]
    acts = {k: synth.random_activations(1, k, seed=k) for k in {s[1] for s in shapes}}
    sample_bytes = sum(w.size for w in weights)
    token_bytes = sum(synth.tensor_bytes(synth.Q4_K, n, k) for _, n, k in llama_linears())

    def one_pass():
        for w, (n, k) in zip(weights, shapes):
            oracle.matmul_t(synth.Q4_K, (1, k, n), acts[k], w)

    one_pass()
    t0 = time.perf_counter()
    reps = 0
    while True:
        one_pass()
        reps += 1
        if time.perf_counter() - t0 > seconds_budget or reps >= 200:
            break
    dt = (time.perf_counter() - t0) / reps
    tok_s = 1.0 / (dt * token_bytes / sample_bytes)
    return {"value": tok_s, "unit": "tok/s", "cores": oracle.threads(), "kind": "port",
            "sample": f"layer-0 linears (7 Q4_K matmuls, {sample_bytes / 1e6:.0f} MB of {token_bytes / 1e9:.2f} GB "
                      f"per token), {reps} passes, scaled by bytes",
            "gbs": sample_bytes / dt / 1e9}


def cpu_moe_sample(cfg, seconds_budget: float = 12.0):
    """Times the oracle on one Qwen3-MoE-shaped layer at batch 1: the Q8_0 attention projections, the f32
    router product and the eight routed experts' Q4_K matmuls, scaled to a token by the layer count plus the
    output head (same kernels, scaled by bytes)."""
    import oracle

    h, inter = cfg.hidden, cfg.moe_inter
    shapes = [(synth.Q8_0, cfg.qkv_rows, h), (synth.Q8_0, h, cfg.q_heads * cfg.head_dim)]
    for _ in range(cfg.n_used):
        shapes += [(synth.Q4_K, inter, h), (synth.Q4_K, inter, h), (synth.Q4_K, h, inter)]
    weights = [synth.random_weight(t, n, k, seed=i) for i, (t, n, k) in enumerate(shapes)]
    acts = {k: synth.random_activations(1, k, seed=k) for k in {s[2] for s in shapes}}
    router = np.random.default_rng(0).standard_normal((cfg.n_expert, h)).astype(np.float32)
    layer_bytes = sum(w.size for w in weights)
    head_bytes = synth.tensor_bytes(synth.Q8_0, cfg.vocab, h)

    def one_layer():
        for w, (t, n, k) in zip(weights, shapes):
            oracle.matmul_t(t, (1, k, n), acts[k], w)
        router @ acts[h][0]

    one_layer()
    t0 = time.perf_counter()
    reps = 0
    while True:
        one_layer()
        reps += 1
        if time.perf_counter() - t0 > seconds_budget or reps >= 400:
            break
    dt = (time.perf_counter() - t0) / reps
    tok_s = 1.0 / (dt * (cfg.layers + head_bytes / layer_bytes))
    return {"value": tok_s, "unit": "tok/s", "cores": oracle.threads(), "kind": "port",
            "sample": f"one layer at batch 1 (2 Q8_0 attention linears, router, {cfg.n_used} experts x 3 Q4_K matmuls, "
                      f"{layer_bytes / 1e6:.0f} MB), {reps} passes, scaled by layers + head bytes"}


def run_reference(args):
    """`--impl reference`: the reference's CPU kernels (C++ oracle port) on this host, all cores.  The figure is
    extrapolated: one layer's matmuls are timed and scaled to a token by bytes (`"extrapolated": true`)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t0 = time.perf_counter()
    budget = max(5.0, min(60.0, 2.0 * (args.steps + args.warmup)))
    if args.workload in ("default", "qwen3moe"):
        from joshua_b200.bench_moe import moe_config
        from joshua_b200.moe_decoder import MoeDecoderConfig

        cfg = MoeDecoderConfig()
        base = cpu_moe_sample(cfg, seconds_budget=budget)
        config = moe_config(cfg, args.batch, args.gpus)
    else:
        base = cpu_llama_sample(seconds_budget=budget)
        config = {"workload": "llama8b_q4k_decode_b1", **LLAMA}
    line = {
        "impl": "reference", "metric": "decode_tok_s", "value": base["value"], "unit": "tok/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 / base["value"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": config, "extrapolated": True,
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line))


# ───────────────────────────── GPU workloads ──────────────────────────────

def cuda_time(fn, steps, warmup, barrier=None):
    """Runs fn() warmup + steps times; returns seconds per step from CUDA events on the current stream."""
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        fn()
    e.record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    return s.elapsed_time(e) * 1e-3 / steps


def run_gemv(args, emit=True):
    import torch

    from joshua_b200.qtensor import QTensor

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    t = TYPE_BY_NAME[args.type]
    n, k, m = args.n, args.k, args.m
    wbytes = synth.tensor_bytes(t, n, k)
    nmat = max(2, int(args.rotate_gb * 1e9 // wbytes))
    bank = synth.random_weight_torch(t, n * nmat, k, 1, dev)
    bank = torch.cat([bank, torch.zeros(16, dtype=torch.uint8, device=dev)])
    ws = [QTensor.from_device(t, bank[i * wbytes:(i + 1) * wbytes]) for i in range(nmat)]
    x = torch.randn(m, k, device=dev)
    y = torch.empty(m, n, device=dev)

    def step():
        for w in ws:
            w.matmul_t_dev((m, k, n), x, y)

    # one CUDA graph over the rotating set: the figure is the kernel's, not the host's launch rate
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        step()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step()
        with ClockSampler(dev.index or 0) as clocks:
            for _ in range(max(3, args.warmup)):
                graph.replay()
            stream.synchronize()
            s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record(stream)
            for _ in range(args.steps):
                graph.replay()
            e0.record(stream)
            stream.synchronize()
        dt = s0.elapsed_time(e0) * 1e-3 / args.steps / nmat
    peak, which = measured_peaks()
    alg = wbytes + 4 * m * (k + n)
    line = {
        "metric": "quant_matmul_gbs", "value": alg / dt / 1e9, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "i8xi8->i32, f32 scales", "data": "synthetic",
        "config": {"workload": f"gemv {args.type} n={n} k={k} m={m}", "rotating_set_gb": nmat * wbytes / 1e9,
                   "l2": "inputs larger than L2", "launch": "one CUDA graph over the rotating set"},
        "roofline": {"bound": "hbm", "achieved": alg / dt / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": alg / dt / 1e9 / peak, "traffic": None, "peak_source": which,
                     "note": "time per matmul includes the activation-plane kernel where one precedes it"},
        "gpu_launches": 2 * nmat * args.steps, "clocks": clocks.summary(),
    }
    del ws, bank
    torch.cuda.empty_cache()
    if emit:
        print(json.dumps(line))
    return line


def run_default(args):
    """The Qwen3-MoE decode step (the workload that shards over GPUs) as the line; on one GPU the dense Llama-8B
    line and the per-format single-matmul figures ride along as `dense` and `kernels`."""
    import copy

    from joshua_b200 import bench_llama, bench_moe

    def extra(line):
        if line["n_gpus"] != 1:
            return
        line["dense"] = bench_llama.run(args, emit=False)
        kernels = []
        for t in ("q4_k", "q8_0", "q2_k", "iq2_xxs", "mxfp4"):
            a = copy.copy(args)
            a.workload, a.type, a.n, a.k, a.m, a.rotate_gb = "gemv", t, 4096, 4096, 1, 0.5
            g = run_gemv(a, emit=False)
            kernels.append({"type": t, "n": 4096, "k": 4096, "m": 1, "gbs": g["value"], "frac_of_hbm": g["roofline"]["frac"],
                            "us_per_matmul": g["ms_per_step"] * 1e3})
        line["kernels"] = kernels

    return bench_moe.run(args, extra=extra)


def run_moe_layer(args):
    """One routed-expert layer at a given token count: the grouped expert matmuls of the MoE configurations
    (MXFP4 384 experts / IQ2_XXS 256 experts / Q4_K 128 experts), device-resident, CUDA events."""
    import torch

    from joshua_b200.moe import GATE_SOFTMAX, Moe, MoeConfig
    from joshua_b200.qtensor import QTensor, default_context

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    t = TYPE_BY_NAME[args.type]
    E, K, h, inter, T = args.experts, args.used, args.k, args.n, args.m
    ctx = default_context(dev.index or 0)
    banks, keep = [], []
    for i, (rows, cols) in enumerate([(inter, h), (inter, h), (h, inter)]):
        nbytes = synth.tensor_bytes(t, E * rows, cols)
        raw = torch.cat([synth.random_weight_torch(t, E * rows, cols, 31 + i, dev), torch.zeros(16, dtype=torch.uint8, device=dev)])
        keep.append(raw)
        banks.append(QTensor.from_device(t, raw[:nbytes], ctx))
    router = (np.random.default_rng(0).standard_normal((E, h)) * 0.5).astype(np.float32)
    layer = Moe(MoeConfig(gating=GATE_SOFTMAX, n_expert=E, n_used=K, hidden=h, inter=inter, norm=True), router, *banks, ctx=ctx)
    layer.reserve(T, T * K)
    # a different token set every call, so that the experts touched change from call to call
    xs = [torch.randn(T, h, device=dev) * 0.02 for _ in range(8)]
    y = torch.empty(T, h, device=dev)
    it = [0]

    def step():
        layer.forward_dev(xs[it[0] % len(xs)], y)
        it[0] += 1

    with ClockSampler(dev.index or 0) as clocks:
        dt = cuda_time(step, args.steps, max(3, args.warmup))
    layer.status()
    per_expert = 2 * synth.tensor_bytes(t, inter, h) + synth.tensor_bytes(t, h, inter)
    # expected number of distinct experts hit by T*K uniform picks
    distinct = E * (1.0 - (1.0 - 1.0 / E) ** (T * K)) if T * K < 50 * E else float(E)
    alg = distinct * per_expert + 8.0 * T * h
    flops = 2.0 * T * K * 3 * h * inter
    peak, which = measured_peaks()
    line = {
        "metric": "moe_layer_tokens_s", "value": T / dt, "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "i8xi8->i32, f32 scales", "data": "synthetic",
        "config": {"workload": f"moe_layer {args.type} E={E} k={K} h={h} inter={inter} tokens={T}",
                   "l2": "expert banks far larger than L2; tokens change every call"},
        "roofline": {"bound": "hbm", "achieved": alg / dt / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": alg / dt / 1e9 / peak, "traffic": None, "peak_source": which,
                     "note": "bytes of the expected number of distinct experts hit, read once",
                     "tflops_algorithmic": flops / dt / 1e12},
        "gpu_launches": 4 * args.steps, "clocks": clocks.summary(),
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="default", choices=["default", "llama8b", "gemv", "qwen3moe", "moe_layer", "mxfp4_experts", "deepseek_v3"])
    ap.add_argument("--tokens", default="1,16,256,4096", help="mxfp4_experts: global token counts of the sweep")
    ap.add_argument("--type", default="q4_k", choices=sorted(TYPE_BY_NAME))
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--rotate-gb", type=float, default=1.0)
    ap.add_argument("--experts", type=int, default=384)
    ap.add_argument("--used", type=int, default=8)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prefill", type=int, default=512)
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.workload == "gemv":
        return run_gemv(args)
    if args.workload == "moe_layer":
        return run_moe_layer(args)
    if args.workload == "default":
        return run_default(args)
    if args.workload == "deepseek_v3":
        from joshua_b200 import bench_deepseek

        return bench_deepseek.run(args)
    if args.workload == "mxfp4_experts":
        from joshua_b200 import bench_experts

        return bench_experts.run(args)
    if args.workload == "qwen3moe":
        from joshua_b200 import bench_moe

        return bench_moe.run(args)
    from joshua_b200 import bench_llama

    return bench_llama.run(args)


if __name__ == "__main__":
    main()
