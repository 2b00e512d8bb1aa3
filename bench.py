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
  strong_scaling  MobileNetV2 topology, 256 images split evenly over the N ranks (the batch-sharded
             configuration of the benchmark), device-resident and end to end
`--impl reference` times that CPU restatement alone with all host threads (the
reference's LLVM toolchain does not exist here, so its own .so cannot be built).
The CPU arm uses the -O3 -march=native build of the restatement; tests keep the -O2 checker.

The timed region is a loop of exactly --steps steps between barriers; the loop is repeated until at
least one second has been timed, and the median loop is reported (`config.loops`).

`--model inner_product --m M --k K --n N [--int8]` times one InnerProduct layer of the sweep
configuration (rows/s; roofline against HBM for M <= 32, where the weights stream, else tensor).
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
    orc.use_fast_library()  # -O3 -march=native build of the same source, compiled on this host
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
                         "sample": f"{sample} single-image calls of the CPU restatement of the reference lowering, "
                                   "gcc -O3 -march=native -ffp-contract=off with OpenMP "
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
    ap.add_argument("--model", default="resnet18",
                    choices=["resnet18", "resnet18_int8", "mobilenet_v2", "single_conv", "inner_product"])
    ap.add_argument("--accuracy-mode", type=int, default=0, help="0 fp32 via split operands, three bf16 MMAs per product (default), 1 tf32, 2 cuda-core fp32")
    ap.add_argument("--gather", action="store_true", help="all-gather the outputs over NCCL inside the timed region")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="budget of the cpu_baseline sample")
    ap.add_argument("--per-layer", default=None, help="write a per-launch roofline table (markdown) to this path")
    ap.add_argument("--min-seconds", type=float, default=1.0, help="repeat the timed loop until this much has been timed")
    ap.add_argument("--no-strong", action="store_true", help="skip the strong_scaling entry (MobileNetV2, 256 images over the ranks)")
    ap.add_argument("--m", type=int, default=256, help="inner_product: rows per step (the batch)")
    ap.add_argument("--k", type=int, default=4096, help="inner_product: input features")
    ap.add_argument("--n", type=int, default=4096, help="inner_product: output features")
    ap.add_argument("--int8", action="store_true", help="inner_product: int8 weights and activations")
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
    f32_dtype = "f32" if args.accuracy_mode == 2 else ("bf16x3" if args.accuracy_mode == 0 else "tf32")
    unit = "images/s"
    if args.model == "resnet18":
        param, bin_ = pkg.zoo.resnet18(os.path.join(tmp, "resnet18"))
        dtype = f32_dtype
    elif args.model == "resnet18_int8":
        param, bin_ = pkg.zoo.resnet18(os.path.join(tmp, "resnet18_int8"), int8=True)
        dtype = "int8"
    elif args.model == "inner_product":
        param, bin_ = pkg.zoo.inner_product(os.path.join(tmp, "ip"), args.k, args.n, int8=args.int8)
        dtype = "int8" if args.int8 else f32_dtype
        args.batch = args.m
        unit = "rows/s"
    else:
        if args.model == "single_conv":
            param, bin_ = pkg.zoo.single_conv(os.path.join(tmp, "single_conv"))
        else:
            param, bin_ = pkg.zoo.mobilenet_v2(os.path.join(tmp, "mobilenet_v2"))
        dtype = f32_dtype
    model = pkg.Model(param, bin_, accuracy_mode=args.accuracy_mode, device=local_rank)
    n = args.batch
    in_shape = model.input_shapes[0]
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")  # > 126 MB of L2
    stream = torch.cuda.current_stream()

    def measure(mdl, count, seed, gather=False, min_seconds=args.min_seconds, sampler=None):
        """Device-resident and end-to-end time of `args.steps` steps of `count` items per rank: the median
        over repeated loops, each loop bracketed by barriers, max over ranks per loop."""
        out_shape = mdl.output_shapes[0]
        gen = torch.Generator(device="cpu").manual_seed(seed + rank)
        x_host = (torch.rand((count, *mdl.input_shapes[0]), generator=gen) * 2 - 1).pin_memory()
        y_host = torch.empty((count, *out_shape)).pin_memory()
        x_dev = x_host.cuda(non_blocking=True)
        y_dev = torch.empty((count, *out_shape), device="cuda")
        gathered = [torch.empty_like(y_dev) for _ in range(world)] if (gather and world > 1) else None

        def step_device():
            mdl.run_device(count, [x_dev.data_ptr()], [y_dev.data_ptr()], stream.cuda_stream)
            if gathered is not None:
                dist.all_gather(gathered, y_dev)

        for _ in range(max(args.warmup, 3)):
            step_device()
        torch.cuda.synchronize()
        if sampler is not None:
            # keep the same load running until nvidia-smi delivers its first sample (bounded)
            wait_until = time.monotonic() + 5.0
            while gathered is None and sampler.proc is not None and sampler.count() == 0 and time.monotonic() < wait_until:
                step_device()
                torch.cuda.synchronize()
        mdl.check_status()

        def one_loop_device():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
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
            return sum(a.elapsed_time(b) for a, b in zip(starts, ends))

        def one_loop_e2e():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(args.steps):
                st = mdl.run_raw(count, [x_host.data_ptr()], [y_host.data_ptr()])
                if st != 0:
                    raise SystemExit(f"ncnn_b200_run_batch failed with status {st}")
            torch.cuda.synchronize()
            return (time.perf_counter() - t0) * 1000.0

        def loops_of(one_loop):
            first = torch.tensor([one_loop()], device="cuda", dtype=torch.float64)
            if world > 1:
                dist.all_reduce(first, op=dist.ReduceOp.MAX)
            # every rank runs the same number of loops: derived from the slowest rank's first loop
            reps = int(min(200, max(1, np.ceil(min_seconds * 1000.0 / max(float(first[0]), 1e-3)))))
            rest = torch.tensor([one_loop() for _ in range(reps - 1)] + [0.0], device="cuda", dtype=torch.float64)
            if world > 1:
                dist.all_reduce(rest, op=dist.ReduceOp.MAX)
            return [float(first[0])] + [float(v) for v in rest[:-1]]

        if sampler is not None:
            sampler.mark_begin()
        dev = loops_of(one_loop_device)
        if sampler is not None:
            sampler.mark_end()
        mdl.check_status()
        for _ in range(2):
            mdl.run_raw(count, [x_host.data_ptr()], [y_host.data_ptr()])
        e2e = loops_of(one_loop_e2e)
        if not torch.isfinite(y_host).all():
            raise SystemExit("non-finite outputs")
        return {"ms_dev": float(np.median(dev)), "ms_e2e": float(np.median(e2e)), "loops": len(dev), "loops_e2e": len(e2e),
                "timed_s": sum(dev) * 1e-3, "h2d": int(x_host.numel() * 4), "d2h": int(y_host.numel() * 4),
                "gathered": gathered is not None}

    sampler = ClockSampler(local_rank)
    sampler.start()
    main_run = measure(model, n, 1234, gather=args.gather, sampler=sampler)
    clocks = sampler.stop()
    ms_dev, ms_e2e = main_run["ms_dev"], main_run["ms_e2e"]

    # the batch-sharded configuration: 256 images of the MobileNetV2 topology split evenly over the ranks
    strong = None
    if not args.no_strong and args.model == "resnet18" and 256 % world == 0 and not args.gather:
        sparam, sbin = pkg.zoo.mobilenet_v2(os.path.join(tmp, "mobilenet_v2_strong"))
        smodel = pkg.Model(sparam, sbin, accuracy_mode=args.accuracy_mode, device=local_rank)
        per_rank = 256 // world
        sr = measure(smodel, per_rank, 4321, min_seconds=0.5)
        strong = {"workload": "mobilenet_v2-topology 3x224x224, 256 images split evenly over the ranks",
                  "images_per_rank": per_rank, "value": 256 * args.steps / (sr["ms_dev"] * 1e-3),
                  "e2e": 256 * args.steps / (sr["ms_e2e"] * 1e-3), "unit": "images/s", "ms_per_step": sr["ms_dev"] / args.steps,
                  "loops": sr["loops"], "scaling": "strong"}
        smodel.close()

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # per-launch timing with CUDA events on the launching stream (same workload, eager launches)
    rows = model.profile(n, repeat=5)
    tc_prefixes = ("tc_gemm_kernel", "tc_gemm2_kernel", "tc_conv_halo_kernel", "tc_stem_kernel", "tc_stem_pool_kernel", "tc_dw_project_kernel", "k_ip_rows")
    tc = [r for r in rows if r["kernel"].startswith(tc_prefixes)]
    peaks = measured_peaks()
    tc_ms = sum(r["ms"] for r in tc)
    tc_flops = sum(r["flops"] for r in tc)
    total_ms = sum(r["ms"] for r in rows)
    achieved = tc_flops / (tc_ms * 1e-3) / 1e12 if tc_ms > 0 else 0.0
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "tc_gemm_dram_traffic.json")
    if args.model == "inner_product":
        workload = f"inner_product M={args.m} K={args.k} N={args.n} {'int8' if args.int8 else 'fp32'}, bias and fused ReLU"
    else:
        workload = f"{args.model}-topology 3x224x224, batch {n} per GPU"
    if os.path.exists(tpath) and args.accuracy_mode == 0:
        with open(tpath) as f:
            entry_ = json.load(f).get(workload)
        if entry_:
            traffic = entry_["dram_bytes_read"] + entry_["dram_bytes_write"]  # bytes per pass, from the ncu capture
    by_kernel = {}
    for r in tc:
        by_kernel[r["kernel"]] = by_kernel.get(r["kernel"], 0.0) + r["ms"]
    names = sorted(by_kernel, key=by_kernel.get, reverse=True)
    # int8 MMAs run at twice the bf16 rate (4.5 POP/s in an MMA-only loop on this pool); no int8 figure is among the
    # measured peaks, so the int8 denominator is twice the measured bf16 one and says so
    int8_work = args.model == "resnet18_int8" or (args.model == "inner_product" and args.int8)
    tensor_peak = peaks["bf16_sustained"] * (2.0 if int8_work else 1.0)
    roofline = {"bound": "tensor", "kernel": "all tensor-core launches of one pass: " + ", ".join(names),
                "achieved": achieved,
                "peak": tensor_peak, "unit": "TOP/s" if int8_work else "TFLOP/s", "frac": achieved / tensor_peak,
                "peak_source": (f"2 x dense bf16 sustained ({peaks['source']}): int8 MMAs issue at twice the bf16 rate" if int8_work
                                else f"dense bf16 sustained, {peaks['source']}"), "traffic": traffic,
                "traffic_note": "DRAM bytes of all tensor-core launches of one pass (ncu, profiles/)" if traffic else None,
                "launches": len(tc), "share_of_step": tc_ms / total_ms if total_ms else None,
                "flops_per_step": tc_flops,
                "ms_by_kernel": {k: round(v, 4) for k, v in by_kernel.items()}}
    if args.model == "inner_product" and args.m <= 32 and tc:
        # weight streaming: the binding roof is HBM (weights + activations + results at storage width)
        algo_bytes = sum(r["bytes"] for r in tc) + args.k * args.n * (1 if args.int8 else 4)
        gbs = algo_bytes / (tc_ms * 1e-3) / 1e9
        roofline.update({"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s", "frac": gbs / peaks["hbm"],
                         "peak_source": f"copy bandwidth, {peaks['source']}", "algorithmic_bytes": algo_bytes})
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
    per_loop = n * world * args.steps
    line = {
        "metric": "images/sec" if unit == "images/s" else "rows/sec", "value": per_loop / (ms_dev * 1e-3), "unit": unit,
        "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_dev / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": {"workload": workload, "accuracy_mode": args.accuracy_mode,
                   "l2": "flushed between timed iterations (256 MB write)", "gather": main_run["gathered"],
                   "loops": main_run["loops"], "timed_seconds": round(main_run["timed_s"], 3),
                   "timing": "median over `loops` loops of exactly `steps` steps, each between barriers, max over ranks"},
        "e2e": {"value": per_loop / (ms_e2e * 1e-3), "unit": unit,
                "h2d_bytes_per_step": main_run["h2d"], "d2h_bytes_per_step": main_run["d2h"], "loops": main_run["loops_e2e"]},
        "gpu_launches": model.launch_count(n) * args.steps,
        "roofline": roofline,
        "cpu_baseline": {"value": cpu_rate, "unit": unit, "cores": os.cpu_count() or 1, "kind": "port",
                         "sample": (f"{cpu_n} single-item calls in {cpu_t:.1f} s of the CPU restatement of the reference "
                                    "lowering, gcc -O3 -march=native -ffp-contract=off with OpenMP") if cpu_n
                         else "not sampled in this run (N > 1 or disabled)"},
        "clocks": clocks,
    }
    if strong is not None:
        line["strong_scaling"] = strong
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
