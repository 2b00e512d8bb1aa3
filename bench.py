#!/usr/bin/env python
"""Throughput benchmark of the B200 runtime on the benchmark's ResNet-18 configuration.

    python bench.py --gpus N --steps K --warmup W            (N = 1)
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...   (N > 1)

One step = one pass of the whole network over a batch of synthetic images on every
rank (weak scaling: --batch images per GPU, no collective on the data path).  Rank 0
prints ONE JSON line:
  value      images/s with the batch already resident in HBM (device-pointer entry,
             CUDA events on the launching stream, L2 flushed between iterations,
             max over ranks)
  e2e        images/s through the host-pointer entry ncnn_b200_run_batch from pinned
             host buffers, copies inside the timed region
  roofline   tensor-core contraction kernel: algorithmic FLOPs / event-timed duration,
             against the measured dense bf16 peak of this pool
  cpu_baseline  the CPU oracle (restatement of the reference lowering) timed on this
             box's host cores on a bounded sample
`--impl reference` times that CPU restatement alone with all host threads (the
reference's LLVM toolchain does not exist here, so its own .so cannot be built).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"bf16_sustained": p.get("bf16_tflops_sustained", 1393.8), "bf16_burst": p.get("bf16_tflops", 1655.3),
                "hbm": p.get("hbm_gbs", 6552.0), "source": "measured"}
    return {"bf16_sustained": 1400.0, "bf16_burst": 1590.0, "hbm": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi.  The process is started before the
    warm-up (nvidia-smi needs a second to come up); every line is stamped on arrival, and the
    summary uses the samples that fell inside the marked window."""

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.samples = []  # (arrival time, line)
        self.t0 = self.t1 = None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.monotonic(), line.strip()))

    def count(self):
        return len(self.samples)

    def mark_begin(self):
        self.t0 = time.monotonic()

    def mark_end(self):
        self.t1 = time.monotonic()

    def in_window(self):
        return sum(1 for t, _ in self.samples if self.t0 is not None and self.t0 <= t <= (self.t1 or time.monotonic()))

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inside = [(t, line) for t, line in self.samples if self.t0 is not None and self.t0 <= t <= self.t1]
        window = "timed region (and the same steps right after it when it was shorter than a sample period)"
        if not inside:
            # e.g. the gather mode, where ranks cannot run extra steps: the warm-up ran the same load
            inside, window = list(self.samples), "warm-up and timed region of the same load"
        for t, line in inside:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons), "window": window}


def use_all_host_threads():
    """torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU baseline is meant to use
    every host core, so the OpenMP runtime of the oracle library is told so explicitly."""
    import ctypes
    cores = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(cores)
    try:
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(cores)
    except OSError:
        pass
    return cores


def cpu_oracle_rate(param, bin_, shape, budget_s, seed=1):
    """images/s of the CPU restatement on this box's cores: a bounded sample of single-image
    calls (the reference has no batch dimension)."""
    use_all_host_threads()
    orc = entry._load_oracle()
    model = orc.Model(param, bin_)
    rng = np.random.default_rng(seed)
    x = rng.uniform(-1, 1, shape).astype(np.float32)
    model.run([x])  # warm-up (also builds the C library)
    t0 = time.perf_counter()
    done = 0
    while True:
        model.run([x])
        done += 1
        el = time.perf_counter() - t0
        if el >= budget_s or done >= 256:
            break
    return done / el, done, el


def run_reference_arm(args, rank, world):
    if rank != 0:
        return
    tmp = tempfile.mkdtemp(prefix="ncnn_b200_bench_")
    pkg = entry.load_package()
    param, bin_ = pkg.zoo.resnet18(os.path.join(tmp, "resnet18"))
    entry._load_oracle().build()
    cores = os.cpu_count() or 1
    per_step = max(4.0, min(20.0, 60.0 / max(args.steps + args.warmup, 1)))
    rates, sample = [], 0
    for i in range(args.warmup + args.steps):
        r, n, el = cpu_oracle_rate(param, bin_, (3, 224, 224), per_step, seed=i)
        if i >= args.warmup:
            rates.append((n, el))
            sample += n
    total_n = sum(n for n, _ in rates)
    total_t = sum(t for _, t in rates)
    value = total_n / total_t
    line = {
        "impl": "reference", "metric": "images/sec", "value": value, "unit": "images/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * total_t / max(args.steps, 1),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "resnet18-topology fp32 224x224, single-image calls (the reference has no batch)"},
        "cpu_baseline": {"value": value, "unit": "images/s", "cores": cores, "kind": "port",
                         "sample": f"{sample} single-image calls of the CPU restatement of the reference lowering "
                                   "(reference LLVM/MLIR 21 toolchain absent: its own .so cannot be built)"},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=64, help="images per GPU per step")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--model", default="resnet18", choices=["resnet18", "resnet18_int8", "mobilenet_v2", "single_conv"])
    ap.add_argument("--accuracy-mode", type=int, default=0, help="0 fp32 via split operands, three bf16 MMAs per product (default), 1 tf32, 2 cuda-core fp32")
    ap.add_argument("--gather", action="store_true", help="all-gather the outputs over NCCL inside the timed region")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="budget of the cpu_baseline sample")
    ap.add_argument("--per-layer", default=None, help="write a per-launch roofline table (markdown) to this path")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the runtime has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if rank == 0:
        entry.build()
    if world > 1:
        dist.barrier()
    pkg = entry.load_package()

    tmp = tempfile.mkdtemp(prefix=f"ncnn_b200_bench_r{rank}_")
    if args.model == "resnet18":
        param, bin_ = pkg.zoo.resnet18(os.path.join(tmp, "resnet18"))
        dtype = "f32" if args.accuracy_mode == 2 else ("bf16x3" if args.accuracy_mode == 0 else "tf32")
    elif args.model == "resnet18_int8":
        param, bin_ = pkg.zoo.resnet18(os.path.join(tmp, "resnet18_int8"), int8=True)
        dtype = "int8"
    else:
        if args.model == "single_conv":
            param, bin_ = pkg.zoo.single_conv(os.path.join(tmp, "single_conv"))
        else:
            param, bin_ = pkg.zoo.mobilenet_v2(os.path.join(tmp, "mobilenet_v2"))
        dtype = "f32" if args.accuracy_mode == 2 else ("bf16x3" if args.accuracy_mode == 0 else "tf32")
    model = pkg.Model(param, bin_, accuracy_mode=args.accuracy_mode, device=local_rank)
    n = args.batch
    in_shape = model.input_shapes[0]
    out_shape = model.output_shapes[0]

    # every rank works on its own shard of the global batch: images are independent
    gen = torch.Generator(device="cpu").manual_seed(1234 + rank)
    x_host = (torch.rand((n, *in_shape), generator=gen) * 2 - 1).pin_memory()
    y_host = torch.empty((n, *out_shape)).pin_memory()
    x_dev = x_host.cuda(non_blocking=True)
    y_dev = torch.empty((n, *out_shape), device="cuda")
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")  # > 126 MB of L2
    stream = torch.cuda.current_stream()
    gathered = [torch.empty_like(y_dev) for _ in range(world)] if (args.gather and world > 1) else None

    def step_device():
        model.run_device(n, [x_dev.data_ptr()], [y_dev.data_ptr()], stream.cuda_stream)
        if gathered is not None:
            dist.all_gather(gathered, y_dev)

    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        step_device()
    torch.cuda.synchronize()
    # keep the same load running until nvidia-smi delivers its first sample (bounded)
    wait_until = time.monotonic() + 5.0
    while gathered is None and sampler.proc is not None and sampler.count() == 0 and time.monotonic() < wait_until:
        step_device()
        torch.cuda.synchronize()
    model.check_status()

    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler.mark_begin()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    for i in range(args.steps):
        flush.fill_(i & 0xff)  # L2 flush between timed iterations
        starts[i].record(stream)
        step_device()
        ends[i].record(stream)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms_dev = sum(s.elapsed_time(e) for s, e in zip(starts, ends))
    # a timed region of a few milliseconds can fall between two samples: the same steps keep
    # running (untimed) until one sample has been taken under this load
    wait_until = time.monotonic() + 2.0
    while gathered is None and sampler.proc is not None and sampler.in_window() == 0 and time.monotonic() < wait_until:
        flush.fill_(0)
        step_device()
        torch.cuda.synchronize()
    sampler.mark_end()
    clocks = sampler.stop()
    model.check_status()

    # end to end through the host-pointer entry: H2D + run + D2H inside the timed call
    for _ in range(2):
        model.run_raw(n, [x_host.data_ptr()], [y_host.data_ptr()])
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        st = model.run_raw(n, [x_host.data_ptr()], [y_host.data_ptr()])
        if st != 0:
            raise SystemExit(f"ncnn_b200_run_batch failed with status {st}")
    torch.cuda.synchronize()
    ms_e2e = (time.perf_counter() - t0) * 1000.0
    if not torch.isfinite(y_host).all():
        raise SystemExit("non-finite outputs")

    times = torch.tensor([ms_dev, ms_e2e], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_dev, ms_e2e = float(times[0]), float(times[1])

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # per-launch timing with CUDA events on the launching stream (same workload, eager launches)
    rows = model.profile(n, repeat=5)
    tc = [r for r in rows if r["kernel"].startswith(("tc_gemm_kernel", "tc_conv_halo_kernel", "tc_stem_kernel"))]
    peaks = measured_peaks()
    tc_ms = sum(r["ms"] for r in tc)
    tc_flops = sum(r["flops"] for r in tc)
    total_ms = sum(r["ms"] for r in rows)
    achieved = tc_flops / (tc_ms * 1e-3) / 1e12 if tc_ms > 0 else 0.0
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "tc_gemm_dram_traffic.json")
    workload = f"{args.model}-topology 3x224x224, batch {n} per GPU"
    if os.path.exists(tpath) and args.accuracy_mode == 0:
        with open(tpath) as f:
            entry_ = json.load(f).get(workload)
        if entry_:
            traffic = entry_["dram_bytes_read"] + entry_["dram_bytes_write"]  # bytes per pass, from the ncu capture
    by_kernel = {}
    for r in tc:
        by_kernel[r["kernel"]] = by_kernel.get(r["kernel"], 0.0) + r["ms"]
    dominant = max(by_kernel, key=by_kernel.get) if by_kernel else None  # the tensor-core kernel with the most time
    roofline = {"bound": "tensor", "kernel": dominant, "achieved": achieved,
                "peak": peaks["bf16_sustained"], "unit": "TFLOP/s", "frac": achieved / peaks["bf16_sustained"],
                "peak_source": f"dense bf16 sustained, {peaks['source']}", "traffic": traffic,
                "traffic_note": "DRAM bytes of all tensor-core launches of one pass (ncu, profiles/)" if traffic else None,
                "launches": len(tc), "share_of_step": tc_ms / total_ms if total_ms else None,
                "flops_per_step": tc_flops}
    if args.per_layer:
        with open(args.per_layer, "w") as f:
            f.write("| kernel | layer | ms | GFLOP | MB | TFLOP/s | GB/s |\n|---|---|---|---|---|---|---|\n")
            for r in rows:
                tf = r["flops"] / (r["ms"] * 1e-3) / 1e12 if r["ms"] > 0 else 0
                gb = r["bytes"] / (r["ms"] * 1e-3) / 1e9 if r["ms"] > 0 else 0
                f.write(f"| {r['kernel']} | {r['layer']} | {r['ms']:.4f} | {r['flops'] / 1e9:.3f} | "
                        f"{r['bytes'] / 1e6:.2f} | {tf:.1f} | {gb:.0f} |\n")

    if args.cpu_seconds > 0 and world == 1:  # the CPU baseline is taken at N = 1 only
        cpu_rate, cpu_n, cpu_t = cpu_oracle_rate(param, bin_, in_shape, args.cpu_seconds)
    else:
        cpu_rate, cpu_n, cpu_t = None, 0, 0.0  # skipped on request (profiling runs)
    total_images = n * world * args.steps
    line = {
        "metric": "images/sec", "value": total_images / (ms_dev * 1e-3), "unit": "images/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_dev / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": {"workload": workload, "accuracy_mode": args.accuracy_mode,
                   "l2": "flushed between timed iterations (256 MB write)", "gather": bool(gathered)},
        "e2e": {"value": total_images / (ms_e2e * 1e-3), "unit": "images/s",
                "h2d_bytes_per_step": int(x_host.numel() * 4), "d2h_bytes_per_step": int(y_host.numel() * 4)},
        "gpu_launches": model.launch_count(n) * args.steps,
        "roofline": roofline,
        "cpu_baseline": {"value": cpu_rate, "unit": "images/s", "cores": os.cpu_count() or 1, "kind": "port",
                         "sample": (f"{cpu_n} single-image calls in {cpu_t:.1f} s of the CPU restatement "
                                    "of the reference lowering") if cpu_n else "not sampled in this run (N > 1 or disabled)"},
        "clocks": clocks,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
