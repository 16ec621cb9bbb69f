#!/usr/bin/env python
"""Benchmark of the causal-attention path: forward + backward TFLOP/s on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg5] [--impl ours|reference]

One "step" is one forward + backward of the whole workload (for N > 1: of this
rank's (batch x head) shard; O and the gradients stay sharded, and the cost of an
optional NCCL all-gather of O is measured separately and reported beside it).  The default workload is the one the headline metric is quoted on:
f16, B=64, T=2048, H=32, head_dim=128 (7.7 TFLOP per step counting causal FLOPs
as 7*B*H*T^2*D).  Rank 0 prints ONE JSON line.

  value      device-timed throughput with inputs resident in HBM (CUDA events, max over ranks)
  e2e        same metric through the C ABI with HOST buffers: pinned host -> device copies of
             Q, K, V, dO and device -> host copies of O, dQ, dK, dV inside the timed region
  roofline   the dominant kernel (the backward main kernel) against the measured dense
             tensor peak in MEASURED_PEAKS.json
  cpu_baseline  the CPU oracle (a C restatement of the reference's CPU path) on a bounded
             sample of (b, h) slices of the same workload, on this box's host cores

--impl reference times that CPU restatement alone (the reference is Rust and cannot be
built in this image), with all host threads, on a bounded sample per step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (dtype, B, T, H, D)
    "cfg1": ("f32", 4, 256, 6, 32),
    "cfg2": ("f16", 8, 1024, 12, 64),
    "cfg4": ("f16", 2, 8192, 16, 128),
    "cfg5": ("f16", 64, 2048, 32, 128),
}
METRIC = "attn_fwd_bwd_tflops"
UNIT = "TFLOP/s"


def flops_fwd_bwd(n_slices: int, T: int, D: int) -> float:
    """Causal fwd+bwd FLOPs, FlashAttention convention: 7 * slices * T^2 * D."""
    return 7.0 * n_slices * T * T * D


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"tflops_burst": p["bf16_tflops"], "tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                "hbm_gbs": p["hbm_gbs"], "source": "measured"}
    return {"tflops_burst": 1590.0, "tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # "under load": samples in the upper half of the power range seen
        thr = (max(power) + min(power)) / 2
        loaded = [c for c, w in zip(sm, power) if w >= thr] or sm
        return {"sm_mhz": statistics.median(loaded), "sm_max_mhz": max(mx), "power_w_max": max(power),
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_baseline(T: int, D: int, n_slices: int, repeats: int):
    """Times the CPU oracle (fwd + bwd, materialising, OpenMP over slices) on `n_slices` slices."""
    import numpy as np
    from oracle import ref
    ref.set_num_threads()                                   # every host core, whatever OMP_NUM_THREADS says
    rng = np.random.default_rng(0)
    base = min(n_slices, 32)
    q, k, v, do = (np.tile(rng.standard_normal((base, 1, T, D), dtype=np.float32), (n_slices // base, 1, 1, 1))
                   for _ in range(4))
    n = q.shape[0]
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        ref.attn_fwd_bwd(q, k, v, do)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return {"value": flops_fwd_bwd(n, T, D) / best / 1e12, "unit": UNIT, "cores": ref.num_threads(), "kind": "port",
            "sample": f"{n} of the workload's (b,h) slices at T={T}, D={D} ({base} distinct seeded N(0,1) slices "
                      f"tiled), fwd+bwd, best of {repeats} runs, {best:.2f} s; f32 C restatement of the reference's "
                      "CPU path (the Rust reference cannot be built here)",
            "seconds": best}


def cpu_sample_size(T: int, D: int, threads: int, target_s: float) -> int:
    # ~0.6 s per (T=2048, D=128) slice per thread measured on a GPU box's host: scale by T^2 * D.
    per = 0.6 * (T / 2048.0) ** 2 * (D / 128.0)
    n = int(target_s * threads / max(per, 1e-6))
    return max(threads, min(n, 4096))


def run_reference(args, dtype, B, T, H, D):
    """--impl reference: the CPU restatement alone, all host threads, bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import ref
    threads = ref.set_num_threads()                         # launchers such as torchrun export OMP_NUM_THREADS=1
    total_budget = 100.0                                    # seconds for the whole run
    n = cpu_sample_size(T, D, threads, total_budget / (args.steps + args.warmup))
    n = max(1, min(n, B * H))
    import numpy as np
    rng = np.random.default_rng(0)
    base = min(n, 32)
    n = n // base * base
    q, k, v, do = (np.tile(rng.standard_normal((base, 1, T, D), dtype=np.float32), (n // base, 1, 1, 1))
                   for _ in range(4))
    for _ in range(args.warmup):
        ref.attn_fwd_bwd(q, k, v, do)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        ref.attn_fwd_bwd(q, k, v, do)
    dt = (time.perf_counter() - t0) / args.steps
    val = flops_fwd_bwd(n, T, D) / dt / 1e12
    sample = (f"{n} of {B * H} (b,h) slices per step (f32 C restatement of the reference CPU path; the workload's "
              f"f16 inputs as f32), {threads} threads")
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(args.workload, dtype, B, T, H, D), "sample": sample},
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def workload_name(name, dtype, B, T, H, D):
    return f"{name}: causal attention fwd+bwd, {dtype}, B={B} T={T} H={H} head_dim={D}, scale 1/sqrt(D)"


def run_rope(args, dtype, B, T, H, D):
    """The pack that feeds the op: rope(q), rope(k) [B,T,H,D] -> [B,H,T,D] and the inverse rotation of
    dQ, dK back to [B,T,H,D]: four launches per step, each reading and writing one tensor once."""
    import numpy as np
    import torch
    from deers_b200 import _lib, ops
    from oracle import ref
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: there is no CPU fallback")
    dev = torch.device("cuda", 0)
    tdtype = torch.float16 if dtype == "f16" else torch.float32
    esize = 2 if dtype == "f16" else 4
    gen = torch.Generator(device=dev).manual_seed(4321)
    xq, xk = (torch.randn(B, T, H, D, device=dev, dtype=torch.float32, generator=gen).to(tdtype) for _ in range(2))
    gq, gk = (torch.randn(B, H, T, D, device=dev, dtype=torch.float32, generator=gen).to(tdtype) for _ in range(2))
    cos, sin = (c.to(dev) for c in ops.precompute_rotary_embeddings(T, D, dtype=tdtype))
    opq, opk = ops.RotaryPack.new(xq, cos, sin), ops.RotaryPack.new(xk, cos, sin)
    ctx = ops.Context.current(dev)

    def step():
        grads = ops.GradientStore()
        opq.forward(); opk.forward()
        opq.backward(grads, gq); opk.backward(grads, gk)

    sampler = ClockSampler(0)
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    ctx.kernel_timing(True)
    launches0 = ctx.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / args.steps
    launches = ctx.launch_count() - launches0
    k_ms, k_n = ctx.kernel_time(_lib.K_ROPE)
    ctx.kernel_timing(False)
    ctx.sync()
    clocks = sampler.stop()
    n = B * T * H * D
    bytes_per_launch = 2.0 * n * esize + 2.0 * T * (D // 2) * esize      # tensor in + out, cache once
    peaks = load_peaks()
    achieved = bytes_per_launch / (k_ms / max(k_n, 1) * 1e-3) / 1e9
    # CPU leg: the C restatement on a bounded sample of batch entries (f32; the f16 path is numpy)
    bs = max(1, min(B, int(2e8 // max(1, T * H * D))))
    xs = np.random.default_rng(0).standard_normal((bs, T, H, D)).astype(np.float32)
    c32, s32 = ref.precompute_rotary_embeddings(T, D)
    ref.rope_pack(xs, c32, s32)
    t0 = time.perf_counter()
    reps = 3
    for _ in range(reps):
        ref.rope_pack(xs, c32, s32)
    cpu_s = (time.perf_counter() - t0) / reps
    cpu_gbs = 2.0 * xs.size * 4 / cpu_s / 1e9
    line = {"metric": "rope_pack_gbs", "value": 4 * bytes_per_launch / (ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
            "config": {"workload": f"{args.workload}: rotary embedding + head-major pack, {dtype}, B={B} T={T} H={H} head_dim={D}",
                       "per_step": "rope(q), rope(k), inverse rope(dq), inverse rope(dk)",
                       "l2": "tensors larger than L2" if n * esize > 126e6 else "tensors fit L2"},
            "gpu_launches": int(launches), "clocks": clocks, "e2e": None,
            "roofline": {"bound": "hbm", "kernel": "rope_pack_kernel", "achieved": achieved, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                         "bytes_per_launch": bytes_per_launch, "avg_launch_ms": k_ms / max(k_n, 1),
                         "peak_source": peaks["source"] + " copy bandwidth"},
            "cpu_baseline": {"value": cpu_gbs, "unit": "GB/s", "cores": ref.num_threads(), "kind": "port",
                             "sample": f"{bs} of {B} batch entries, f32 C restatement of apply_rotary_emb + permute, "
                                       f"{cpu_s:.3f} s per pass"}}
    print(json.dumps(line))


def run_rmsnorm(args, B, T, H, D):
    """RMSNorm forward + backward over [B*T, H*D] f32 (src/nn.rs:244-251): 8 + 12 bytes per element."""
    import numpy as np
    import torch
    from deers_b200 import _lib, ops
    from oracle import ref
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: there is no CPU fallback")
    dev = torch.device("cuda", 0)
    rows, C = B * T, H * D
    gen = torch.Generator(device=dev).manual_seed(77)
    x = torch.randn(rows, C, device=dev, generator=gen)
    dy = torch.randn(rows, C, device=dev, generator=gen)
    ctx = ops.Context.current(dev)
    small = rows * C * 4 < 126e6
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if small else None

    def step():
        op = ops.RMSNorm.new(x, 1e-6)
        op.forward()
        op.backward(ops.GradientStore(), dy)

    sampler = ClockSampler(0)
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    ctx.kernel_timing(True)
    launches0 = ctx.launch_count()
    total_ms = 0.0
    for _ in range(args.steps):
        if flush is not None:
            flush.zero_()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        step()
        ev1.record()
        torch.cuda.synchronize()
        total_ms += ev0.elapsed_time(ev1)
    ms = total_ms / args.steps
    launches = ctx.launch_count() - launches0
    k_ms, k_n = ctx.kernel_time(_lib.K_NORM)
    ctx.kernel_timing(False)
    ctx.sync()
    clocks = sampler.stop()
    bytes_step = rows * C * 4.0 * 5 + rows * 4.0 * 2
    peaks = load_peaks()
    achieved = bytes_step / (k_ms / args.steps * 1e-3) / 1e9
    sr = max(1, min(rows, int(5e7 // C)))
    xs = np.random.default_rng(0).standard_normal((sr, C)).astype(np.float32)
    ref.rmsnorm(xs, 1e-6, xs)
    t0 = time.perf_counter()
    ref.rmsnorm(xs, 1e-6, xs)
    cpu_s = time.perf_counter() - t0
    line = {"metric": "rmsnorm_fwd_bwd_gbs", "value": bytes_step / (ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.workload}: RMSNorm forward + backward, f32, rows={rows} C={C}",
                       "l2": "256 MB flush write between steps" if small else "tensors larger than L2"},
            "gpu_launches": int(launches), "clocks": clocks, "e2e": None,
            "roofline": {"bound": "hbm", "kernel": "rmsnorm_kernel (forward + backward)", "achieved": achieved,
                         "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                         "bytes_per_step": bytes_step, "kernel_ms_per_step": k_ms / args.steps,
                         "peak_source": peaks["source"] + " copy bandwidth"},
            "cpu_baseline": {"value": sr * C * 4.0 * 5 / cpu_s / 1e9, "unit": "GB/s", "cores": ref.num_threads(),
                             "kind": "port", "sample": f"{sr} of {rows} rows, f32 C restatement, {cpu_s:.3f} s"}}
    print(json.dumps(line))


def run_decode(args, dtype, B, T, H, D):
    """One sampling step with a KV cache: q [B,H,1,D] against K, V [B,H,T,D]; reads K and V once."""
    import numpy as np
    import torch
    from deers_b200 import _lib, ops
    from oracle import ref
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: there is no CPU fallback")
    dev = torch.device("cuda", 0)
    tdtype = torch.float16 if dtype == "f16" else torch.float32
    esize = 2 if dtype == "f16" else 4
    gen = torch.Generator(device=dev).manual_seed(31)
    k, v = (torch.randn(B, H, T, D, device=dev, dtype=torch.float32, generator=gen).to(tdtype) for _ in range(2))
    q = torch.randn(B, H, 1, D, device=dev, dtype=torch.float32, generator=gen).to(tdtype)
    ctx = ops.Context.current(dev)
    small = 2 * B * H * T * D * esize < 126e6
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if small else None
    sampler = ClockSampler(0)
    for _ in range(max(args.warmup, 3)):
        ops.attention_decode(q, k, v)
    torch.cuda.synchronize()
    ctx.kernel_timing(True)
    launches0 = ctx.launch_count()
    total_ms = 0.0
    for _ in range(args.steps):
        if flush is not None:
            flush.zero_()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        ops.attention_decode(q, k, v)
        ev1.record()
        torch.cuda.synchronize()
        total_ms += ev0.elapsed_time(ev1)
    ms = total_ms / args.steps
    launches = ctx.launch_count() - launches0
    k_ms, k_n = ctx.kernel_time(_lib.K_DECODE)
    ctx.kernel_timing(False)
    ctx.sync()
    clocks = sampler.stop()
    bytes_step = 2.0 * B * H * T * D * esize
    peaks = load_peaks()
    achieved = bytes_step / (k_ms / args.steps * 1e-3) / 1e9
    ns = max(1, min(B * H, int(2e8 // (T * D))))
    ks = np.random.default_rng(0).standard_normal((1, ns, T, D)).astype(np.float32)
    qs = np.random.default_rng(1).standard_normal((1, ns, 1, D)).astype(np.float32)
    ref.attn_decode(qs, ks, ks)
    t0 = time.perf_counter()
    ref.attn_decode(qs, ks, ks)
    cpu_s = time.perf_counter() - t0
    line = {"metric": "attn_decode_tokens_per_s", "value": B / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
            "config": {"workload": f"{args.workload}: decode attention, one new token per slice, {dtype}, B={B} H={H} "
                                   f"cache T={T} head_dim={D}",
                       "l2": "256 MB flush write between steps" if small else "cache larger than L2"},
            "gpu_launches": int(launches), "clocks": clocks, "e2e": None,
            "roofline": {"bound": "hbm", "kernel": "decode_partial_kernel + decode_combine_kernel", "achieved": achieved,
                         "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                         "bytes_per_step": bytes_step, "kernel_ms_per_step": k_ms / args.steps,
                         "peak_source": peaks["source"] + " copy bandwidth"},
            "cpu_baseline": {"value": 2.0 * ns * T * D * 4 / cpu_s / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
                             "sample": f"{ns} of {B * H} slices, numpy f32 restatement, {cpu_s:.3f} s"}}
    print(json.dumps(line))


def run_gemm(args):
    """Linear forward y = x W on the tcgen05 GEMM, with torch.matmul (cuBLAS) timed beside it for context."""
    import numpy as np
    import torch
    from deers_b200 import _lib, ops
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: there is no CPU fallback")
    M, N, K = (int(v) for v in args.gemm.split(","))
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn(M, K, device=dev, generator=gen).to(torch.float16)
    w = (torch.randn(K, N, device=dev, generator=gen) / K ** 0.5).to(torch.float16)
    ctx = ops.Context.current(dev)
    op = ops.Linear.new(x, w)
    sampler = ClockSampler(0)
    for _ in range(max(args.warmup, 3)):
        op.forward()
    torch.cuda.synchronize()
    ctx.kernel_timing(True)
    launches0 = ctx.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        op.forward()
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / args.steps
    launches = ctx.launch_count() - launches0
    k_ms, k_n = ctx.kernel_time(_lib.K_GEMM)
    ctx.kernel_timing(False)
    ctx.sync()
    clocks = sampler.stop()
    for _ in range(3):
        torch.matmul(x, w)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        torch.matmul(x, w)
    e1.record()
    torch.cuda.synchronize()
    lib_ms = e0.elapsed_time(e1) / args.steps
    flops = 2.0 * M * N * K
    peaks = load_peaks()
    achieved = flops / (k_ms / max(k_n, 1) * 1e-3) / 1e12
    xs, ws_ = x[:min(M, 2048)].float().cpu().numpy(), w.float().cpu().numpy()
    t0 = time.perf_counter()
    xs @ ws_
    cpu_s = time.perf_counter() - t0
    line = {"metric": "gemm_f16_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"Linear forward y[{M},{N}] = x[{M},{K}] W[{K},{N}], f16 in / f32 accumulate / f16 out",
                       "l2": "operands larger than L2" if (M * K + K * N + M * N) * 2 > 126e6 else "operands fit L2",
                       "library_gemm_tflops_for_context": flops / (lib_ms * 1e-3) / 1e12},
            "gpu_launches": int(launches), "clocks": clocks, "e2e": None,
            "roofline": {"bound": "tensor", "kernel": "gemm_f16_kernel", "achieved": achieved, "peak": peaks["tflops_burst"],
                         "unit": "TFLOP/s", "frac": achieved / peaks["tflops_burst"], "traffic": None,
                         "flops_per_launch": flops, "avg_launch_ms": k_ms / max(k_n, 1),
                         "peak_source": peaks["source"] + " burst bf16 (kernel timed alone)"},
            "cpu_baseline": {"value": 2.0 * xs.shape[0] * N * K / cpu_s / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(),
                             "kind": "port", "sample": f"{xs.shape[0]} of {M} rows, numpy f32 matmul, {cpu_s:.3f} s"}}
    print(json.dumps(line))


def run_block(args, B, T, H, D):
    """The attention block of src/models/gpt.rs:118-147 in f16 on this library's kernels, forward + backward."""
    import torch
    from deers_b200 import _lib, ops
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: there is no CPU fallback")
    dev = torch.device("cuda", 0)
    C = H * D
    gen = torch.Generator(device=dev).manual_seed(17)
    h16 = lambda *shape, s=1.0: (torch.randn(*shape, device=dev, generator=gen) * s).to(torch.float16)
    x, dy = h16(B, T, C), h16(B, T, C)
    wqkv, wo = h16(C, 3 * C, s=C ** -0.5), h16(C, C, s=C ** -0.5)
    cos, sin = (c.to(dev) for c in ops.precompute_rotary_embeddings(T, D, dtype=torch.float16))
    ctx = ops.Context.current(dev)
    ws = torch.empty(max(ops.workspace_bytes(torch.empty(B, H, T, D, dtype=torch.float16, device=dev), pass_=2), 256),
                     dtype=torch.uint8, device=dev)

    def step():
        lin_qkv = ops.Linear.new(x, wqkv)
        qkv = lin_qkv.forward()
        q4, k4, v4 = (qkv[..., i * C:(i + 1) * C].view(B, T, H, D) for i in range(3))
        rq, rk = ops.RotaryPack.new(q4, cos, sin), ops.RotaryPack.new(k4, cos, sin)
        qh, kh, vh = rq.forward(), rk.forward(), v4.permute(0, 2, 1, 3)
        att = ops.CausalAttention.new(qh, kh, vh, token_major_out=True)
        o = att.forward()
        y_att = o.permute(0, 2, 1, 3).reshape(B, T, C)
        lin_o = ops.Linear.new(y_att, wo)
        lin_o.forward()
        grads = ops.GradientStore()
        lin_o.backward(grads, dy)
        d_att = grads.get(y_att).view(B, T, H, D).permute(0, 2, 1, 3)
        dqkv = torch.empty_like(qkv)
        dq4, dk4, dv4 = (dqkv[..., i * C:(i + 1) * C].view(B, T, H, D) for i in range(3))
        dqh, dkh, _ = ops.attention_bwd(qh, kh, vh, att.o, att.lse, d_att, att.scale, True, workspace=ws,
                                        dv_out=dv4.permute(0, 2, 1, 3))
        rq.backward(grads, dqh, dx_out=dq4)
        rk.backward(grads, dkh, dx_out=dk4)
        lin_qkv.backward(grads, dqkv)

    sampler = ClockSampler(0)
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    ctx.kernel_timing(True)
    launches0 = ctx.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / args.steps
    launches = ctx.launch_count() - launches0
    kinds = (("gemm", _lib.K_GEMM), ("rope", _lib.K_ROPE), ("attn_fwd", _lib.K_FWD), ("attn_bwd_prep", _lib.K_BWD_PREP),
             ("attn_bwd_dkdv", _lib.K_BWD_MAIN), ("attn_bwd_dq", _lib.K_BWD_DQ))
    kernels = {name: ctx.kernel_time(kind)[0] / args.steps for name, kind in kinds}
    ctx.kernel_timing(False)
    ctx.sync()
    clocks = sampler.stop()
    tokens = B * T
    gemm_flops = 3 * 2.0 * tokens * C * (3 * C + C)                 # forward, dgrad, wgrad of both projections
    attn_flops = flops_fwd_bwd(B * H, T, D)
    peaks = load_peaks()
    achieved = (gemm_flops + attn_flops) / (sum(kernels.values()) * 1e-3) / 1e12
    line = {"metric": "attention_block_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"{args.workload}: attention block forward + backward, f16, B={B} T={T} H={H} head_dim={D} "
                                   f"(C={C}): fused qkv GEMM, rotary pack, causal attention, output projection",
                       "flops_per_step": gemm_flops + attn_flops, "gemm_flops": gemm_flops, "attention_flops": attn_flops,
                       "l2": "tensors larger than L2" if tokens * C * 2 > 126e6 else "tensors fit L2"},
            "gpu_launches": int(launches), "clocks": clocks, "e2e": None, "kernels_ms_per_step": kernels,
            "roofline": {"bound": "tensor", "kernel": "all kernels of the block", "achieved": achieved,
                         "peak": peaks["tflops_sustained"], "unit": "TFLOP/s", "frac": achieved / peaks["tflops_sustained"],
                         "traffic": None, "peak_source": peaks["source"] + " sustained bf16"},
            "cpu_baseline": None}
    print(json.dumps(line))


def run_adamw(args):
    """One optimizer step of the reference's training loop: gradient norm, clip, AdamW over every parameter
    (src/optim.rs:214-297), fused into three kinds of launches."""
    import numpy as np
    import torch
    from deers_b200 import _lib, ops
    from oracle import ref
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: there is no CPU fallback")
    dev = torch.device("cuda", 0)
    # GPT of the reference's README config: wte, 6 x (q, k, v, out proj, fc, proj), lm_head
    shapes = [(50257, 192)] + [(192, 192)] * 4 * 6 + [(192, 768), (768, 192)] * 6 + [(50257, 192)]
    gen = torch.Generator(device=dev).manual_seed(99)
    params = [torch.randn(s, device=dev, generator=gen) for s in shapes]
    glist = [torch.randn(s, device=dev, generator=gen) for s in shapes]
    n_elem = sum(p.numel() for p in params)
    opt = ops.AdamW(params, lr=6e-4, betas=(0.9, 0.95), weight_decay=0.1)
    ctx = ops.Context.current(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)     # 88 MB of state fits L2: flush between steps

    def step():
        grads = ops.GradientStore()
        for p, g in zip(params, glist):
            grads.insert(p, g)
        norm = ops.grad_norm_device(params, grads)
        opt.step_with_grads(grads, clip_norm=norm, max_norm=1.0)

    sampler = ClockSampler(0)
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    ctx.kernel_timing(True)
    launches0 = ctx.launch_count()
    total_ms = 0.0
    for _ in range(args.steps):
        flush.zero_()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        step()
        ev1.record()
        torch.cuda.synchronize()
        total_ms += ev0.elapsed_time(ev1)
    ms = total_ms / args.steps
    launches = ctx.launch_count() - launches0
    k_ms, k_n = ctx.kernel_time(_lib.K_OPTIM)
    ctx.kernel_timing(False)
    ctx.sync()
    clocks = sampler.stop()
    bytes_step = n_elem * 4.0 * (1 + 7)            # norm pass reads g; step reads w, g, m, v and writes w, m, v
    peaks = load_peaks()
    achieved = bytes_step / (k_ms / args.steps * 1e-3) / 1e9
    # CPU leg: the C restatement over the same tensors (clip + step), all host threads
    hw = [p.cpu().numpy().reshape(-1).copy() for p in params]
    hg = [g.cpu().numpy().reshape(-1).copy() for g in glist]
    hm, hv = [np.zeros_like(w) for w in hw], [np.zeros_like(w) for w in hw]
    t0 = time.perf_counter()
    gs = [g.copy() for g in hg]
    ref.clip_grad_norm(gs, 1.0)
    for w, g, m, v in zip(hw, gs, hm, hv):
        ref.adamw_step(w, g, m, v, 1, 6e-4, (0.9, 0.95), 1e-8, 0.1)
    cpu_s = time.perf_counter() - t0
    line = {"metric": "adamw_clip_step_params_per_s", "value": n_elem / (ms * 1e-3), "unit": "parameters/s", "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"gradient norm + clip + AdamW over {len(shapes)} tensors, {n_elem} f32 parameters "
                                   "(the reference's GPT: vocab 50257, n_embd 192, 6 layers)",
                       "l2": "256 MB flush write between steps (88 MB of state would otherwise stay in L2)"},
            "gpu_launches": int(launches), "clocks": clocks, "e2e": None,
            "roofline": {"bound": "hbm", "kernel": "grad_sq_sum_kernel + grad_norm_kernel + adamw_kernel",
                         "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                         "traffic": None, "bytes_per_step": bytes_step, "kernel_ms_per_step": k_ms / args.steps,
                         "peak_source": peaks["source"] + " copy bandwidth"},
            "cpu_baseline": {"value": n_elem / cpu_s, "unit": "parameters/s", "cores": ref.num_threads(), "kind": "port",
                             "sample": f"the whole step once, f32 C restatement of clip_grad_norm + AdamW, {cpu_s:.3f} s"}}
    print(json.dumps(line))


GPT_CFG3 = {"vocab": 50257, "n_layer": 6, "n_head": 6, "n_embd": 192, "mlp": 768, "B": 4, "T": 256,
            "eps": 1e-5, "rope_base": 10000.0, "lr": 5e-4, "wd": 0.1, "max_grad_norm": 1.0}


def gpt_workload_name():
    c = GPT_CFG3
    return (f"cfg3: GPT training step, f32, {c['n_layer']} layers, {c['n_head']} heads, n_embd {c['n_embd']}, mlp "
            f"{c['mlp']}, vocab {c['vocab']}, RMSNorm eps {c['eps']}, RoPE base {c['rope_base']:g}; B={c['B']} "
            f"T={c['T']}, ids uniform in [0, vocab); cross_entropy + clip_grad_norm({c['max_grad_norm']}) + "
            f"AdamW(lr={c['lr']}, wd={c['wd']})")


def gpt_gemm_flops():
    c = GPT_CFG3
    n, C, Hm, V = c["B"] * c["T"], c["n_embd"], c["mlp"], c["vocab"]
    linear = c["n_layer"] * (4 * C * C + 2 * C * Hm) + C * V
    return 6.0 * n * linear                                 # forward + two backward products per Linear


def gpt_cpu_step(params, ids, tgt, moments, step):
    """One whole training step on the CPU oracle: forward, loss, backward, clip, AdamW.  Returns seconds."""
    from oracle import ref
    c = GPT_CFG3
    t0 = time.perf_counter()
    r = ref.gpt_step((c["vocab"], c["n_layer"], c["n_head"], c["n_embd"], c["mlp"]), params, ids, tgt,
                     eps=c["eps"], rope_base=c["rope_base"], want_logits=False)
    ref.clip_grad_norm(r["grads"], c["max_grad_norm"])
    for p, g, (m, v) in zip(params, r["grads"], moments):
        ref.adamw_step(p, g, m, v, step, c["lr"], weight_decay=c["wd"])
    return time.perf_counter() - t0, r["loss"]


def run_gpt_reference(args):
    """--impl reference --workload cfg3: the CPU restatement of the whole step, all host threads."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import numpy as np
    from oracle import ref
    threads = ref.set_num_threads()
    c = GPT_CFG3
    cfg = (c["vocab"], c["n_layer"], c["n_head"], c["n_embd"], c["mlp"])
    params = ref.gpt_init_params(cfg, seed=0)
    moments = [(np.zeros_like(p), np.zeros_like(p)) for p in params]
    rng = np.random.default_rng(1)
    ids = rng.integers(0, c["vocab"], (c["B"], c["T"]))
    tgt = rng.integers(0, c["vocab"], c["B"] * c["T"])
    steps = max(1, min(args.steps, 5))                      # a step takes seconds on the host: bounded
    warm = min(args.warmup, 1)
    for i in range(warm):
        gpt_cpu_step(params, ids, tgt, moments, i + 1)
    total = 0.0
    for i in range(steps):
        dt, _ = gpt_cpu_step(params, ids, tgt, moments, warm + i + 1)
        total += dt
    dt = total / steps
    val = c["B"] * c["T"] / dt
    sample = (f"the whole step (B*T = {c['B'] * c['T']} tokens) {steps} time(s) after {warm} warm-up: f32 C restatement "
              f"of the reference CPU path (forward, cross-entropy, backward, clip, AdamW), {threads} threads")
    line = {"impl": "reference", "metric": "gpt_step_tok_per_s", "value": val, "unit": "tok/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": gpt_workload_name(), "sample": sample},
            "cpu_baseline": {"value": val, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def run_gpt_step(args):
    """--workload cfg3: the f32 GPT training step of BASELINE cfg 3 on one GPU (N > 1: one independent replica
    per rank, weak scaling, no collective: the reference has no data-parallel training)."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from deers_b200 import _lib, gpt
    from oracle import ref
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: there is no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    c = GPT_CFG3
    cfg = (c["vocab"], c["n_layer"], c["n_head"], c["n_embd"], c["mlp"])
    B, T = c["B"], c["T"]
    params = ref.gpt_init_params(cfg, seed=0)               # numpy draws from the reference's init distributions
    model = gpt.GPT(gpt.GPTConfig(c["vocab"], T, c["n_layer"], c["n_head"], c["n_embd"], c["mlp"], c["eps"],
                                  c["rope_base"]), dev, B)
    model.load_parameters(params)
    if args.no_graph:
        model.set_graph(False)
    rng = np.random.default_rng(1 + rank)
    n_batches = 8                                            # rotate batches so no step repeats the previous one's ids
    ids_h = [rng.integers(0, c["vocab"], (B, T)) for _ in range(n_batches)]
    tgt_h = [rng.integers(0, c["vocab"], B * T) for _ in range(n_batches)]
    ids_d = [torch.from_numpy(a).to(dev) for a in ids_h]
    tgt_d = [torch.from_numpy(a).to(dev) for a in tgt_h]
    kw = dict(lr=c["lr"], weight_decay=c["wd"], max_grad_norm=c["max_grad_norm"])
    ctx = model.ctx

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local) if rank == 0 else None
    torch.cuda.synchronize()
    torch.cuda.set_stream(model.stream)                     # the timed loop and its events live on the model's stream
    for i in range(max(args.warmup, 3)):
        model.train_step(ids_d[i % n_batches], tgt_d[i % n_batches], **kw)
    barrier()
    # The driver fixes --steps; a block of K steps lasts milliseconds here, so the block is repeated until two
    # seconds of device time have passed and the median block is reported.
    blocks = []
    launches0 = ctx.launch_count()
    while sum(blocks) < 2000.0 and len(blocks) < 2000:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for i in range(args.steps):
            loss_d, norm_d = model.train_step(ids_d[i % n_batches], tgt_d[i % n_batches], **kw)
        ev1.record()
        torch.cuda.synchronize()
        blocks.append(ev0.elapsed_time(ev1))
    barrier()
    launches = (ctx.launch_count() - launches0) / len(blocks)
    graph_active = model.graph_active()
    clocks = sampler.stop() if sampler else None
    ms = statistics.median(blocks) / args.steps
    ms_t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms_t, op=dist.ReduceOp.MAX)
    ms_max = float(ms_t.item())
    final_loss = float(loss_d.item())

    # ---- e2e: ids and targets from host memory, the loss read back, every step
    e_steps = max(args.e2e_steps, 5)
    model.train_step_host(ids_h[0], tgt_h[0], **kw)
    barrier()
    t0 = time.perf_counter()
    for i in range(e_steps):
        model.train_step_host(ids_h[i % n_batches], tgt_h[i % n_batches], **kw)
    e_ms = torch.tensor([(time.perf_counter() - t0) * 1e3 / e_steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(e_ms, op=dist.ReduceOp.MAX)
    e2e = {"value": world * B * T / (float(e_ms.item()) * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": 2 * B * T * 8,
           "d2h_bytes_per_step": 8, "ms_per_step": float(e_ms.item()), "steps": e_steps,
           "api": "deers_b200_gpt_train_step_host: int64 ids and targets from host memory, loss and gradient norm read "
                  "back, one blocking call per step (host clock)"}

    # ---- per-kernel-family device times: a few eager steps (no graph) bracketed by events
    model.set_graph(False)
    model.train_step(ids_d[0], tgt_d[0], **kw)
    torch.cuda.synchronize()
    ctx.kernel_timing(True)
    k_steps = 3
    l0 = ctx.launch_count()
    for i in range(k_steps):
        model.train_step(ids_d[i % n_batches], tgt_d[i % n_batches], **kw)
    eager_launches = (ctx.launch_count() - l0) / k_steps
    fams = {"gemm_f32": _lib.K_GEMM, "gemm_f16x3_head": _lib.K_GEMM_X3, "attn_fwd_f32": _lib.K_FWD, "attn_bwd_delta_f32": _lib.K_BWD_PREP,
            "attn_bwd_f32 (dK/dV and dQ blocks in one launch)": _lib.K_BWD_MAIN, "rope_pack": _lib.K_ROPE,
            "rmsnorm": _lib.K_NORM, "embedding_cross_entropy": _lib.K_GPT, "grad_norm_adamw": _lib.K_OPTIM}
    kernels = {}
    for name, kind in fams.items():
        t_ms, n = ctx.kernel_time(kind)
        kernels[name] = {"launches_per_step": n / k_steps, "ms_per_step": t_ms / k_steps}
    ctx.kernel_timing(False)
    ctx.sync()
    model.set_graph(not args.no_graph)

    if rank == 0:
        peaks = load_peaks()
        # Two GEMM families: the head (lm_head forward, its weight and input gradients: 3 products of
        # 2 * 1024 * 50257 * 192 FLOPs) on the tensor core as split-f16 products, and the 72 products of the blocks on
        # the FFMA pipe.  The roofline entry is the family that takes longer.
        n_tok, C_, Hm_, V_ = c["B"] * c["T"], c["n_embd"], c["mlp"], c["vocab"]
        head_flops = 6.0 * n_tok * C_ * V_
        block_flops = 6.0 * n_tok * c["n_layer"] * (4 * C_ * C_ + 2 * C_ * Hm_)
        head_ms = kernels["gemm_f16x3_head"]["ms_per_step"]
        block_ms = kernels["gemm_f32"]["ms_per_step"]
        sm_max = (clocks or {}).get("sm_max_mhz") or 1965.0
        ffma_peak = 148 * 128 * 2 * sm_max * 1e6 / 1e12      # FFMA lanes x 2 flops x clock
        at_max_clock = bool(clocks and clocks.get("sm_mhz") and clocks["sm_mhz"] >= 0.95 * sm_max and
                            "sw_power_cap" not in clocks.get("reasons", []))
        tc_peak = peaks["tflops_burst" if at_max_clock else "tflops_sustained"]
        head = {"bound": "tensor", "kernel": "gemm_f16x3_kernel + split / reduce (lm_head forward, wgrad, dgrad)",
                "achieved": head_flops / (head_ms * 1e-3) / 1e12 if head_ms else None, "peak": tc_peak, "unit": "TFLOP/s",
                "frac": (head_flops / (head_ms * 1e-3) / 1e12 / tc_peak) if head_ms else None,
                # DRAM bytes per step of the three products, the two splits and the reduction, from the ncu capture of
                # this very workload (profiles/gpt_step_cfg3_kernels.md); None at other model sizes
                "traffic": 725.0e6 if (n_tok, C_, V_) == (1024, 192, 50257) else None,
                "flops_per_step": head_flops, "kernel_ms_per_step": head_ms,
                "note": "algorithmic f32 FLOPs; the kernel executes three f16 products per f32 product",
                "peak_source": f"{peaks['source']} {'burst' if at_max_clock else 'sustained'} bf16"}
        block = {"bound": "fp32 FFMA pipe (the reference computes these products in full f32, CUBLAS_COMPUTE_32F)",
                 "kernel": "gemm_f32_kernel (the 72 Linear forward / dgrad / wgrad products of the blocks)",
                 "achieved": block_flops / (block_ms * 1e-3) / 1e12 if block_ms else None, "peak": ffma_peak, "unit": "TFLOP/s",
                 "frac": (block_flops / (block_ms * 1e-3) / 1e12 / ffma_peak) if block_ms else None,
                 # DRAM bytes per step: 72 launches x 2.24 MB, the mean of the four forward shapes captured by ncu at this
                 # workload (operands and results live in L2; profiles/gpt_step_cfg3_kernels.md); None at other sizes
                 "traffic": 161.0e6 if (n_tok, C_, Hm_, c["n_layer"]) == (1024, 192, 768, 6) else None,
                 "flops_per_step": block_flops, "kernel_ms_per_step": block_ms,
                 "peak_source": f"148 SMs x 128 FFMA lanes x 2 x {sm_max:.0f} MHz (nominal; MEASURED_PEAKS.json holds no f32 figure)"}
        roofline = dict(head if head_ms >= block_ms else block)
        roofline["other_family"] = block if head_ms >= block_ms else head
        cb = None
        if not args.no_cpu_baseline:
            threads = ref.set_num_threads()
            cpu_params = [p.copy() for p in params]
            moments = [(np.zeros_like(p), np.zeros_like(p)) for p in cpu_params]
            dt, _ = gpt_cpu_step(cpu_params, ids_h[0], tgt_h[0], moments, 1)
            dt2, _ = gpt_cpu_step(cpu_params, ids_h[1], tgt_h[1], moments, 2)
            dt = min(dt, dt2)
            cb = {"value": B * T / dt, "unit": "tok/s", "cores": threads, "kind": "port", "seconds": dt,
                  "sample": "the whole step (1024 tokens) twice, best taken: f32 C restatement of the reference CPU path "
                            "(forward, cross-entropy, backward, clip, AdamW)"}
        line = {"metric": "gpt_step_tok_per_s", "value": world * B * T / (ms_max * 1e-3), "unit": "tok/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_max, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": gpt_workload_name(), "parameters": 21952896,
                           "weights": "seeded draws from the reference's init distributions (uniform +-1/sqrt(in), normal embedding)",
                           "parallelism": "1 GPU" if world == 1 else f"{world} independent replicas (replicas only)",
                           "timing": f"median of {len(blocks)} blocks of {args.steps} steps ({sum(blocks) / 1e3:.2f} s of device time)",
                           "l2": "weights, moments, gradients and logits (560 MB) exceed L2: no flush needed",
                           "final_loss": final_loss,
                           "graph": ("forward + loss + backward + gradient norm replayed from a CUDA graph, AdamW launched after it"
                                     if graph_active else "not captured: every kernel launched eagerly"),
                           "ms_x_median_sm_mhz": (ms_max * clocks["sm_mhz"]) if clocks and clocks.get("sm_mhz") else None},
                "e2e": e2e, "gpu_launches": int(round(eager_launches * args.steps)),
                "launches_per_step": {"kernels": eager_launches, "host_calls_with_graph": launches / args.steps},
                "clocks": clocks, "roofline": roofline, "kernels": kernels, "cpu_baseline": cb}
        sys.stdout.flush()
        os.write(real_stdout, (json.dumps(line) + "\n").encode())
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="cfg5", choices=sorted(WORKLOADS) + ["cfg3"],
                    help="cfg1/2/4/5: attention forward + backward (TFLOP/s); cfg3: the f32 GPT training step (tok/s)")
    ap.add_argument("--shape", default=None, help="B,T,H,D: a custom shape (profiling captures on a small case)")
    ap.add_argument("--dtype", default=None, choices=["f16", "f32"], help="dtype for --shape")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--gather", default="auto", choices=["auto", "peer", "nccl", "none"],
                    help="N>1: the all-gather of O that the sharded workload names, inside the timed step.  peer "
                         "(default): the C ABI's copy-engine pushes into every rank's buffer, started after the forward "
                         "and overlapping the backward; nccl: a library all-gather on a side stream; none: O stays "
                         "sharded (compute only).  The other variants are timed beside it under config.gather_probe")
    ap.add_argument("--bwd", default="keep-ds", choices=["keep-ds", "recompute"],
                    help="f16 backward: keep the dS tiles in the workspace between its kernels (default), or "
                         "recompute S and dP in the dQ kernel (workspace of a few MB)")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--e2e-chunk-mb", type=int, default=128,
                    help="input bytes (Q,K,V,dO together) per chunk of the pipelined host call, in MiB")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true",
                    help="cfg3: launch every kernel of the step eagerly instead of replaying the captured graph "
                         "(what a per-kernel profiler capture wants)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--rope", action="store_true",
                    help="time the fused rotary embedding + head-major pack (q and k, forward and inverse) "
                         "on the workload's shape instead of attention; 1 GPU")
    ap.add_argument("--rmsnorm", action="store_true",
                    help="time the fused RMSNorm forward + backward on [B*T, H*D] f32 rows of the workload; 1 GPU")
    ap.add_argument("--decode", action="store_true",
                    help="time decode-time attention (one new token per slice against a cache of T rows) on the "
                         "workload's B, H, T, head_dim instead of the training step; 1 GPU")
    ap.add_argument("--gemm", default=None, metavar="M,N,K",
                    help="time the tcgen05 f16 GEMM y[M,N] = x[M,K] W[K,N] (Linear forward) instead of attention; 1 GPU")
    ap.add_argument("--block", action="store_true",
                    help="time the whole f16 attention block (fused qkv GEMM, rotary pack, attention, output projection) "
                         "forward + backward on the workload's B, T, H, head_dim; 1 GPU")
    ap.add_argument("--adamw", action="store_true",
                    help="time the fused multi-tensor AdamW step with the gradient-norm clip on the parameter "
                         "shapes of the reference's GPT (22 M parameters in 38 tensors) instead of attention; 1 GPU")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.workload == "cfg3":
        if args.impl == "reference":
            run_gpt_reference(args)
        else:
            run_gpt_step(args)
        return
    dtype, B, T, H, D = WORKLOADS[args.workload]
    if args.shape:
        B, T, H, D = (int(x) for x in args.shape.split(","))
        dtype = args.dtype or "f16"
        args.workload = "custom"
    if args.rope:
        run_rope(args, dtype, B, T, H, D)
        return
    if args.adamw:
        run_adamw(args)
        return
    if args.rmsnorm:
        run_rmsnorm(args, B, T, H, D)
        return
    if args.decode:
        run_decode(args, dtype, B, T, H, D)
        return
    if args.gemm:
        run_gemm(args)
        return
    if args.block:
        run_block(args, B, T, H, D)
        return
    if args.impl == "reference":
        run_reference(args, dtype, B, T, H, D)
        return

    import torch
    import torch.distributed as dist
    from deers_b200 import _lib, ops, shard

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
        args.gpus = world
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: there is no CPU fallback for the attention path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    # Libraries (NCCL's version banner) may write to stdout: point fd 1 at stderr for the run and keep
    # the real stdout for the one JSON line.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    tdtype = torch.float16 if dtype == "f16" else torch.float32
    esize = 2 if dtype == "f16" else 4
    n_total = B * H
    begin, end = shard.partition(n_total, world, rank)
    n_local = end - begin
    Bs, Hs = shard.shard_shape(B, H, world, rank)
    scale = ops.default_scale(D)

    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    q, k, v, do = (torch.randn(Bs, Hs, T, D, device=dev, dtype=torch.float32, generator=gen).to(tdtype)
                   for _ in range(4))
    ctx = ops.Context.current(dev)
    # The backward keeps its dS tiles when the workspace has room for them (pass 2), else recomputes S and dP.
    ws_bytes = ops.workspace_bytes(q, scale, pass_=1 if args.bwd == "recompute" else 2)
    workspace = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
    nccl_gather = shard.OverlappedGather(n_total, T, D, tdtype, dev) if world > 1 else None
    # Two gather buffers, used by alternate steps: the pushes of step i then have until the end of step i + 1
    # (whose forward writes the other buffer) to leave, a whole step instead of one backward.  At 8 GPUs a rank
    # sends 7/8 of a GB per step, which takes longer than its backward.
    peer_gather, peer_gather_b, peer_error = None, None, None
    if world > 1:
        try:
            peer_gather = shard.PeerGather(n_total, T, D, tdtype, dev, ctx)
            peer_gather_b = shard.PeerGather(n_total, T, D, tdtype, dev, ctx)
        except Exception as err:                             # peer mappings unavailable on this box: say so, use NCCL
            peer_error = f"{type(err).__name__}: {err}"
        ok = torch.tensor([1 if peer_gather_b is not None else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)            # all ranks take the same path
        if int(ok.item()) == 0:
            peer_gather = peer_gather_b = None
    peer_pair = (peer_gather, peer_gather_b)
    step_no = [0]

    gather_mode = args.gather if world > 1 else "none"
    if gather_mode in ("peer", "auto") and peer_gather is None:
        gather_mode = "nccl"
    gather_choice = None                                     # filled in by --gather auto

    def step(mode=None):
        mode = gather_mode if mode is None else mode
        if mode == "peer":
            # the forward writes this rank's O straight into its slices of this step's gather buffer
            pg, pg_prev = peer_pair[step_no[0] & 1], peer_pair[(step_no[0] & 1) ^ 1]
            step_no[0] += 1
            o, lse = ops.attention_fwd(q, k, v, scale, True, out=pg.local().view(Bs, Hs, T, D))
            pg.start()                                       # pushes run on the copy engines under the following kernels
        else:
            o, lse = ops.attention_fwd(q, k, v, scale, True)
            if mode == "nccl":
                nccl_gather.start(o)
        grads = ops.attention_bwd(q, k, v, o, lse, do, scale, True, workspace=workspace)
        if mode == "peer":
            pg_prev.join()                                   # the previous step's pushes have left: its buffer is free again
        elif mode == "nccl":
            nccl_gather.finish()
        return o, grads

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local) if rank == 0 else None     # started early: nvidia-smi needs a moment
    auto_gather = gather_mode == "auto"
    if auto_gather:
        gather_mode = "peer"                                 # warm up on the peer path; the choice follows below
    for _ in range(args.warmup):
        step()
    barrier()

    # The driver fixes --steps; a block of K steps can be far shorter than the time the clocks need to settle under
    # the power cap, so blocks are repeated (every rank the same number of times) until about two seconds of device
    # time have passed, and the median block is reported.  Per-kernel events are taken in one extra block.
    def timed_block(mode=None, steps=None):
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        a.record()
        for _ in range(steps or args.steps):
            step(mode)
        if (gather_mode if mode is None else mode) == "peer":
            for pg in peer_pair:                             # every push of the block ends inside the timed region
                pg.join()
        b_.record()
        barrier()
        t = torch.tensor([a.elapsed_time(b_) / (steps or args.steps)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)         # max over ranks
        return float(t.item())

    if auto_gather:
        # Which all-gather of O rides best beside the kernels depends on the number of GPUs: the copy-engine pushes
        # one after the other or all of a rank's world - 1 at once, or the library all-gather.  Each candidate runs
        # five blocks of the same step; the quickest one is then timed.
        candidates = [("peer", lanes) for lanes in sorted({1, world - 1})] + [("nccl", None)]
        results, setting = {}, {}
        for mode, lanes in candidates:
            if lanes:
                for pg in peer_pair:
                    pg.set_lanes(lanes)
            name = mode + (f"_lanes{lanes}" if lanes else "")
            # whole blocks, like the timed ones: the first few steps of a gather run faster than its steady state
            results[name] = statistics.median([timed_block(mode) for _ in range(5)])
            setting[name] = (mode, lanes)
        picked = min(results, key=results.get)               # the same on every rank: the times are maxima over ranks
        gather_mode, lanes = setting[picked]
        if lanes:
            for pg in peer_pair:
                pg.set_lanes(lanes)
        gather_choice = {"step_ms": results, "picked": picked}
    first = timed_block()
    n_blocks = int(min(400, max(3, round(2000.0 / max(first * args.steps, 1e-3)))))
    launches0 = ctx.launch_count()
    blocks = [timed_block() for _ in range(n_blocks)]
    launches = (ctx.launch_count() - launches0) // n_blocks
    ms_max = statistics.median(blocks)
    ctx.kernel_timing(True)
    timed_block()
    ktimes = {name: ctx.kernel_time(kind) for name, kind in
              (("fwd", _lib.K_FWD), ("bwd_prep", _lib.K_BWD_PREP), ("bwd_main", _lib.K_BWD_MAIN),
               ("bwd_dq", _lib.K_BWD_DQ))}
    ctx.kernel_timing(False)
    ctx.sync()
    clocks = sampler.stop() if sampler else None

    # ---- N > 1: what the optional all-gather of O costs (overlapped with the backward, and alone) ----
    gather_probe = None
    if world > 1:
        probe = {"bytes_received_per_gpu": (n_total - n_local) * T * D * esize,
                 "bytes_sent_per_gpu": (world - 1) * n_local * T * D * esize, "peer_error": peer_error}
        modes = ["none", "nccl"] + (["peer"] if peer_gather is not None else [])
        for mode in modes:
            step(mode)
            probe[f"step_ms_gather_{mode}"] = statistics.median([timed_block(mode, 5) for _ in range(5)])

        def alone(fn):
            a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            a.record()
            for _ in range(5):
                fn()
            b_.record()
            barrier()
            t = torch.tensor([a.elapsed_time(b_) / 5], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        o_probe, _ = ops.attention_fwd(q, k, v, scale, True)
        probe["nccl_allgather_alone_ms"] = alone(lambda: shard.gather_output(o_probe, n_total, out=nccl_gather.out))
        if peer_gather is not None:
            def push():
                peer_gather.start()
                peer_gather.join()
            probe["peer_allgather_alone_ms"] = alone(push)
            # gathered O must equal what the library all-gather delivers (every rank's forward is deterministic)
            o_p, _ = ops.attention_fwd(q, k, v, scale, True, out=peer_gather.local().view(Bs, Hs, T, D))
            peer_gather.start()
            got = peer_gather.wait_all()
            want = shard.gather_output(o_p, n_total, out=nccl_gather.out)
            torch.cuda.synchronize()
            probe["peer_gather_matches_nccl"] = bool(torch.equal(got, want))
        gather_probe = probe
        del o_probe
    total_flops = flops_fwd_bwd(n_total, T, D)
    value = total_flops / (ms_max * 1e-3) / 1e12

    # ---- e2e: host tensors through the C ABI's pipelined host call, copies inside the timed region ----
    e2e = None
    if not args.no_e2e:
        host_in = [torch.empty(t.shape, dtype=tdtype, pin_memory=True) for t in (q, k, v, do)]
        for h_, d_ in zip(host_in, (q, k, v, do)):
            h_.copy_(d_)
        host_out = tuple(torch.empty(q.shape, dtype=tdtype, pin_memory=True) for _ in range(4)) + \
                   (torch.empty(q.shape[:3], dtype=torch.float32, pin_memory=True),)
        nbytes = q.numel() * esize
        chunk = max(1, min(n_local, (args.e2e_chunk_mb << 20) // max(4 * T * D * esize, 1)))
        chunk = max(1, min(chunk, -(-n_local // 12)))        # at least twelve chunks: the three-stage pipeline needs a run-in
        dsc = _lib.AttnDesc()
        _lib.lib().deers_b200_attn_desc_compact(dsc, Bs, Hs, T, D, _lib.F16 if dtype == "f16" else _lib.F32, 1, scale)
        scratch = torch.empty(int(_lib.lib().deers_b200_attn_host_scratch_bytes(dsc, chunk)), dtype=torch.uint8, device=dev)

        def e2e_step():
            ops.attention_fwd_bwd_host(*host_in, scale, True, chunk_slices=chunk, device=dev, scratch=scratch, out=host_out)

        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            e2e_step()                                       # returns when the last device->host copy is done
        torch.cuda.synchronize()
        e_ms = torch.tensor([(time.perf_counter() - t0) * 1e3 / args.e2e_steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(e_ms, op=dist.ReduceOp.MAX)
        e2e = {"value": total_flops / (float(e_ms.item()) * 1e-3) / 1e12, "unit": UNIT,
               "h2d_bytes_per_step": 4 * nbytes, "d2h_bytes_per_step": 4 * nbytes + q.numel() // D * 4,
               "ms_per_step": float(e_ms.item()), "steps": args.e2e_steps,
               "host_link_gbs_each_way_per_gpu": 4 * nbytes / (float(e_ms.item()) * 1e-3) / 1e9,
               "chunks_per_rank": -(-n_local // chunk),
               "api": f"deers_b200_attn_fwd_bwd_host: pinned host Q,K,V,dO -> O,dQ,dK,dV,lse on the host, "
                      f"{chunk} slices per chunk, copies and kernels pipelined on three streams; timed on the host "
                      "clock around the blocking calls (the call returns after the last copy)"}
        del host_in, host_out, scratch

    if rank == 0:
        peaks = load_peaks()
        bwd_ms, bwd_n = ktimes["bwd_main"]
        bwd_avg = bwd_ms / max(bwd_n, 1)
        # The dominant kernel is the dK/dV kernel: 4 causal products (S^T, dP^T, dV, dK) of n*T^2*D FLOPs each.
        dkdv_flops = 4.0 * n_local * T * T * D
        # Which measured peak is the honest comparator follows from the clocks seen during the timed region: at
        # (nearly) the maximum clock with no power cap the burst figure, otherwise the sustained one.
        at_max_clock = bool(clocks and clocks.get("sm_mhz") and clocks.get("sm_max_mhz") and
                            clocks["sm_mhz"] >= 0.95 * clocks["sm_max_mhz"] and "sw_power_cap" not in clocks.get("reasons", []))
        peak_kind = "burst" if at_max_clock else "sustained"
        peak = peaks["tflops_" + peak_kind] if dtype == "f16" else None
        roofline = None
        if dtype == "f16":
            achieved = dkdv_flops / (bwd_avg * 1e-3) / 1e12
            # DRAM traffic of this kernel from an ncu capture of a small case (the 128 slices of B=8, H=16 at
            # T=2048, D=128: 922.3 MB when it also writes the dS tiles, 376.0 MB when it does not; summaries
            # under profiles/), scaled by the slices one launch processes; traffic is proportional to the
            # slice count.
            per128 = 376.0e6 if args.bwd == "recompute" else 922.3e6
            traffic = per128 / 128 * n_local if (T == 2048 and D == 128) else None
            roofline = {"bound": "tensor", "kernel": "attn_bwd_dkdv_f16_kernel", "achieved": achieved, "peak": peak,
                        "unit": UNIT, "frac": achieved / peak, "traffic": traffic,
                        "flops_per_launch": dkdv_flops,
                        "peak_source": f"{peaks['source']} {peak_kind} bf16 (median SM clock {clocks.get('sm_mhz') if clocks else None} MHz "
                                       f"of {clocks.get('sm_max_mhz') if clocks else None}, reasons {clocks.get('reasons') if clocks else None})",
                        "frac_of_burst": achieved / peaks["tflops_burst"], "frac_of_sustained": achieved / peaks["tflops_sustained"],
                        "avg_launch_ms": bwd_avg}
        else:
            # f32 FFMA path at this size is HBM/latency bound: algorithmic bytes of the whole step.
            alg_bytes = 12.0 * n_local * T * D * esize + 3.0 * n_local * T * 4
            kms = sum(v_[0] for v_ in ktimes.values()) / max(args.steps, 1)
            achieved = alg_bytes / (kms * 1e-3) / 1e9
            roofline = {"bound": "hbm", "kernel": "attn f32 fwd + bwd kernels", "achieved": achieved,
                        "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                        "peak_source": f"{peaks['source']} copy bandwidth"}
        fwd_ms, fwd_n = ktimes["fwd"]
        kernels = {name: {"launches": n_, "avg_ms": (ms_ / n_ if n_ else None)} for name, (ms_, n_) in ktimes.items()}
        if dtype == "f16":
            # causal tile products per kernel
            for name, nprod in (("fwd", 2.0), ("bwd_main", 4.0), ("bwd_dq", 3.0 if args.bwd == "recompute" else 1.0)):
                ms_, n_ = ktimes[name]
                if n_:
                    kernels[name]["tflops_executed"] = nprod * n_local * T * T * D / (ms_ / n_ * 1e-3) / 1e12
        cb = None
        if not args.no_cpu_baseline:
            from oracle import ref
            threads = ref.set_num_threads()
            n_cpu = cpu_sample_size(T, D, threads, 12.0)
            n_cpu = max(1, min(n_cpu, n_total))
            n_cpu = max(32, n_cpu // 32 * 32) if n_cpu >= 32 else n_cpu
            cb = cpu_baseline(T, D, n_cpu, repeats=1)
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_max, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": dtype, "data": "synthetic",
                "config": {"workload": workload_name(args.workload, dtype, B, T, H, D),
                           "flops_per_step": total_flops, "flop_convention": "7*B*H*T^2*D (causal fwd 2, bwd 5)",
                           "parallelism": f"(b x h) shards over {world} GPU(s), {n_local} slices on rank 0",
                           "gather": ({"peer": "all-gather of O inside the timed step: copy-engine pushes (deers_b200_allgather_o) from two alternating buffers, overlapping the backward and the next forward; all pushes of a block are joined before its closing timestamp",
                                       "nccl": "all-gather of O inside the timed step: NCCL on a side stream, overlapping the backward",
                                       "none": "none (compute only)"}[gather_mode] if world > 1 else "n/a (1 GPU)"),
                           "gather_choice": gather_choice,
                           "gather_probe": gather_probe,
                           "timing": f"median of {n_blocks} blocks of {args.steps} steps ({sum(blocks) * args.steps / 1e3:.2f} s of device time), max over ranks per block",
                           "ms_x_median_sm_mhz": (ms_max * clocks["sm_mhz"]) if clocks and clocks.get("sm_mhz") else None,
                           "backward": ("dS tiles kept in the workspace between the dK/dV and dQ kernels"
                                        if args.bwd == "keep-ds" and dtype == "f16" else "dQ kernel recomputes S and dP"),
                           "workspace_bytes": ws_bytes,
                           "l2": "inputs larger than L2 (no flush needed)" if 4 * q.numel() * esize > 126e6
                                 else "inputs fit in L2 (not flushed)",
                           "frac_of_dense_peak": value / world / peaks["tflops_" + peak_kind],
                           "frac_of_burst_peak": value / world / peaks["tflops_burst"],
                           "frac_of_sustained_peak": value / world / peaks["tflops_sustained"],
                           "peak_tflops": peaks["tflops_" + peak_kind], "peak_kind": peak_kind, "peak_source": peaks["source"]},
                "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "roofline": roofline,
                "kernels": kernels, "cpu_baseline": cb}
        sys.stdout.flush()
        os.write(real_stdout, (json.dumps(line) + "\n").encode())
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
