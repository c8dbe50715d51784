#!/usr/bin/env python
"""Headline benchmark: flash-attention forward throughput on B200.

  python bench.py --gpus N --steps K --warmup W            (native arm)
  python bench.py --impl reference --gpus N --steps K ...  (CPU reference arm)

A "step" is one pass of the hot path over one batch of synthetic input: one
fa_fwd_bf16 launch on this rank's shard. At N = 1 the workload is the headline
configuration (B=4, H=16, S=4096, D=128, non-causal, bf16, N(0,1) inputs). At N > 1
each rank holds one such shard of a batch N times larger, split by
(batch x head) with no collective on the data path ("weak" scaling); one process
per GPU, launched by torch.distributed.run.

Prints ONE JSON line on rank 0. `value` is whole-job TFLOPS with inputs resident
in HBM, timed with CUDA events on the launching stream, max over ranks. `e2e` is
the same metric through the library call with HOST buffers: pinned host -> device
copies of Q, K, V and the device -> host copy of O inside the timed region;
`e2e.grouped_kv` repeats it with K and V shared by groups of four query heads
(same flops, half the bytes in).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "attention fwd TFLOPS (bf16, fp32 accumulate), B=4 H=16 S=4096 D=128 per GPU"
WORKLOADS = {
    # name: (B, H, S, D, causal, sigma_qk, seed)
    "c2": (4, 16, 4096, 128, False, 1.0, 20260002),
    "c3": (16, 16, 2048, 64, False, 1.0, 20260003),
    "c4": (8, 32, 8192, 128, True, 0.5, 20260004),
}
GEMM_WORKLOADS = {"c5": (8192, 8192, 8192, 20260005)}   # M, N (per GPU), K, seed; entries U[-1,1]
# Row-wise fp32 neighbours of the attention path (not headline configurations; HBM-bound, reported in
# GB/s of algorithmic bytes): name -> (rows, N, seed); 1 GiB in, 1 GiB out per launch.
ROWWISE_WORKLOADS = {"softmax": (65536, 4096, 20260011), "rms_norm": (65536, 4096, 20260012),
                     "layer_norm": (65536, 4096, 20260013), "swiglu": (65536, 4096, 20260014)}
# DRAM traffic of one launch (dram__bytes_read.sum + dram__bytes_write.sum) from the
# ncu captures summarised in profiles/fa_fwd_d128_c2.md, profiles/fa_fwd_c3_c4.md and
# profiles/gemm_bf16_c5.md.
# (softmax: captured at rows = 16384 and scaled by 4 to the bench's 65536 rows, every row being
# read and written once: profiles/rowwise_softmax_n4096.md)
NCU_TRAFFIC_BYTES = {"c2": 201.44e6 + 43.03e6, "c3": 201.39e6 + 45.83e6, "c4": 1649.54e6 + 517.57e6,
                     "c5": 1067.3e6 + 131.1e6,
                     "softmax": 4 * (268.45e6 + 218.52e6)}
FALLBACK_PEAK_TFLOPS = 1590.0
FALLBACK_PEAK_GBS = 6650.0


def host_threads():
    """Host cores usable by this process (torchrun pins OMP_NUM_THREADS=1, so the CPU
    legs ask the oracle for this many threads explicitly)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def attn_flops(B, H, S, D, causal):
    return (2.0 if causal else 4.0) * B * H * S * S * D


def rowwise_cpu(workload, x, w, b):
    """The oracle's float64 restatement of the reference's CPU reference for `workload`."""
    import oracle
    if workload == "softmax":
        return oracle.softmax_ref_numpy(x)
    if workload == "rms_norm":
        return oracle.rms_norm_ref_numpy(x, w, 1e-6)
    if workload == "layer_norm":
        return oracle.layer_norm_ref_numpy(x, w, b, 1e-5)
    return oracle.swiglu_ref_numpy(x, w)


def rowwise_cpu_sample(workload, sample_rows):
    """Times the numpy oracle on `sample_rows` rows of the workload (one thread)."""
    import numpy as np
    rows, N, seed = ROWWISE_WORKLOADS[workload]
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((sample_rows, N)).astype(np.float32)
    w = rng.standard_normal(N).astype(np.float32) if workload != "swiglu" else \
        rng.standard_normal((sample_rows, N)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    t = time.perf_counter()
    rowwise_cpu(workload, x, w, b)
    dt = time.perf_counter() - t
    nbytes = (3 if workload == "swiglu" else 2) * sample_rows * N * 4
    return nbytes / dt / 1e9, dt


class ClockSampler(threading.Thread):
    """Samples the SM clock (every ~0.3 ms) and the throttle reasons and board power (every
    8th sample) through NVML for the life of the run; each sample carries its host time, so any timed
    region can ask for the clocks it saw. Reads only: no GPU setting is changed."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index = index
        self.t = []          # perf_counter of each sample
        self.mhz = []
        self.reason_log = []  # (perf_counter, frozenset of active reasons)
        self.power_log = []   # (perf_counter, board power in watts)
        self.max_mhz = None
        self.power_limit_w = None
        self.error = None
        self._stop_evt = threading.Event()

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            try:
                self.power_limit_w = nv.nvmlDeviceGetEnforcedPowerLimit(h) / 1000.0
            except Exception:
                self.power_limit_w = None
            names = {
                "hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown,
                "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown,
                "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap,
            }
            i = 0
            while not self._stop_evt.is_set():
                self.mhz.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                self.t.append(time.perf_counter())
                if i % 8 == 0:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                    self.reason_log.append((self.t[-1], frozenset(k for k, bit in names.items() if r & bit)))
                    try:
                        self.power_log.append((self.t[-1], nv.nvmlDeviceGetPowerUsage(h) / 1000.0))
                    except Exception:
                        pass
                i += 1
                time.sleep(0.0003)
        except Exception as e:  # NVML missing: report that instead of inventing numbers
            self.error = f"nvml_unavailable:{type(e).__name__}"

    def stop(self):
        self._stop_evt.set()

    def window(self, t0, t1):
        """Clock summary of the samples taken between two perf_counter times."""
        n = len(self.mhz)     # the lists only grow; read a consistent prefix
        vals = [self.mhz[i] for i in range(n) if t0 <= self.t[i] <= t1]
        reasons = set()
        for t, rs in list(self.reason_log):
            if t0 <= t <= t1:
                reasons |= rs
        if self.error:
            reasons.add(self.error)
        watts = [w for t, w in list(self.power_log) if t0 <= t <= t1]
        return {"sm_mhz": statistics.median(vals) if vals else None,
                "sm_mhz_min": min(vals) if vals else None, "sm_max_mhz": self.max_mhz,
                "samples": len(vals), "reasons": sorted(reasons),
                "power_w": statistics.median(watts) if watts else None,
                "power_w_max": max(watts) if watts else None, "power_limit_w": self.power_limit_w}


def physical_gpu_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


def bind_to_gpu_local_cpus(index, pci_bus_id=None):
    """Multi-GPU runs: run this rank on the CPUs NVML reports as local to its GPU, so the
    pinned host buffers of the end-to-end leg (first touched by this process) sit on
    the GPU's own NUMA node and eight ranks do not push their copies over one socket
    link. Returns how many CPUs the rank ended up with, or None if nothing was changed."""
    try:
        import pynvml
        pynvml.nvmlInit()
        handle = (pynvml.nvmlDeviceGetHandleByPciBusId(pci_bus_id.encode()) if pci_bus_id
                  else pynvml.nvmlDeviceGetHandleByIndex(index))
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        local = {64 * w + b for w, word in enumerate(words) for b in range(64) if (word >> b) & 1}
        allowed = os.sched_getaffinity(0)
        pick = local & allowed
        if len(pick) >= 2 and pick != allowed:
            os.sched_setaffinity(0, pick)
            return len(pick)
    except Exception:
        pass
    return None


# --------------------------------------------------------------------------- CPU arm
def run_reference_arm(args):
    """The reference's own CPU implementation of the path (its Julia CPU checker
    restated in C: no Julia toolchain exists on these machines), all host threads.
    Each step is a bounded sample of the workload: 1-4 (batch, head) slices, sized
    from one timed slice so that warmup + steps stay near two minutes."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    import oracle
    oracle.build_c_oracle()
    if args.workload in ROWWISE_WORKLOADS:
        rows, N, seed = ROWWISE_WORKLOADS[args.workload]
        sample_rows = 4096
        for _ in range(min(args.warmup, 1)):
            rowwise_cpu_sample(args.workload, sample_rows)
        vals = [rowwise_cpu_sample(args.workload, sample_rows) for _ in range(min(args.steps, 20))]
        gbs = statistics.median(v[0] for v in vals)
        dt = statistics.median(v[1] for v in vals)
        sample = f"{sample_rows} of {rows} rows of N={N} per step, numpy float64 restatement of the reference's CPU reference"
        print(json.dumps({
            "impl": "reference", "metric": f"{args.workload} GB/s (fp32 in, fp32 out, algorithmic bytes)",
            "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": len(vals), "warmup": min(args.warmup, 1),
            "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f64", "data": "synthetic", "config": {"workload": f"{args.workload}: rows={rows} N={N}", "sample": sample},
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": 1, "kind": "port", "sample": sample},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}), flush=True)
        return
    if args.workload in GEMM_WORKLOADS:
        # bounded sample: a 512 x 512 block of C over the full K (the reference's _ghb_cpu_ref)
        M, N, K, seed = GEMM_WORKLOADS[args.workload]
        rng = np.random.default_rng(seed)
        a, bt = (oracle.to_bf16_bits((rng.random((512, K)) * 2 - 1).astype(np.float32)) for _ in range(2))
        for _ in range(min(args.warmup, 2)):
            oracle.gemm_ref_c(a, bt, nthreads=host_threads())
        t0 = time.perf_counter()
        for _ in range(args.steps):
            oracle.gemm_ref_c(a, bt, nthreads=host_threads())
        dt = (time.perf_counter() - t0) / args.steps
        tflops = 2.0 * 512 * 512 * K / dt / 1e12
        sample = f"512 x 512 block of C over K={K} per step"
        print(json.dumps({
            "impl": "reference", "metric": "GEMM TFLOPS (bf16 in, fp32 accumulate), M=N=K=8192 per GPU",
            "value": tflops, "unit": "TFLOPS", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": {"workload": f"{args.workload}: M={M} N={N} K={K}", "sample": sample},
            "cpu_baseline": {"value": tflops, "unit": "TFLOPS", "cores": host_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": tflops, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}), flush=True)
        return
    B, H, S, D, causal, sigma, seed = WORKLOADS[args.workload]
    rng = np.random.default_rng(seed)
    q, k, v = (oracle.to_bf16_bits((rng.standard_normal((4, S, D)) * s).astype(np.float32))
               for s in (sigma, sigma, 1.0))
    scale = 1.0 / math.sqrt(D)
    t = time.perf_counter()
    oracle.attention_ref_c(q[:1], k[:1], v[:1], scale, causal, nthreads=host_threads())
    t_slice = time.perf_counter() - t
    n_slices = int(max(1, min(4, 120.0 / (max(args.steps + args.warmup, 1) * t_slice))))
    for _ in range(args.warmup):
        oracle.attention_ref_c(q[:n_slices], k[:n_slices], v[:n_slices], scale, causal, nthreads=host_threads())
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.attention_ref_c(q[:n_slices], k[:n_slices], v[:n_slices], scale, causal, nthreads=host_threads())
    dt = (time.perf_counter() - t0) / args.steps
    tflops = attn_flops(1, n_slices, S, D, causal) / dt / 1e12
    threads = host_threads()
    sample = f"{n_slices} of {B * H} (batch, head) slices of S={S} D={D} per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: B={B} H={H} S={S} D={D} causal={causal}", "sample": sample},
        "cpu_baseline": {"value": tflops, "unit": "TFLOPS", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference arm = C port of the reference's CPU checker (fab_cpu_ref) on the host cores; "
                "PTX.jl's own GPU kernels need Julia + CUDA.jl, which this box does not have",
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- native arm
def peaks():
    """(burst bf16 TF/s, sustained bf16 TF/s, HBM GB/s, 'measured' | 'fallback')."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            mp = json.load(f)
        return (float(mp["bf16_tflops"]), float(mp.get("bf16_tflops_sustained", mp["bf16_tflops"])),
                float(mp["hbm_gbs"]), "measured")
    except Exception:
        return FALLBACK_PEAK_TFLOPS, 1400.0, FALLBACK_PEAK_GBS, "fallback"


class Problem:
    """One workload resident on this rank's GPU: inputs, output, the launch, its work."""

    def __init__(self, name, inputs, out, run, work, algo_bytes, text):
        self.name, self.inputs, self.out, self.run = name, inputs, out, run
        self.work, self.algo_bytes, self.text = work, algo_bytes, text


def attention_problem(ops, dev, name, seed_offset=0):
    import torch
    B, H, S, D, causal, sigma, seed = WORKLOADS[name]
    g = torch.Generator(device=dev).manual_seed(seed + seed_offset)
    q = (torch.randn(B, H, S, D, device=dev, generator=g) * sigma).to(torch.bfloat16)
    k = (torch.randn(B, H, S, D, device=dev, generator=g) * sigma).to(torch.bfloat16)
    v = torch.randn(B, H, S, D, device=dev, generator=g).to(torch.bfloat16)
    o = torch.empty_like(q)
    sm_scale = 1.0 / math.sqrt(D)

    def run(ins, out, stream=None):
        ops.fa_fwd(ins[0], ins[1], ins[2], causal=causal, sm_scale=sm_scale, out=out, stream=stream)

    return Problem(name, [q, k, v], o, run, attn_flops(B, H, S, D, causal), 4 * q.numel() * 2,
                   f"{name}: B={B} H={H} S={S} D={D} causal={causal}")


def attention_shard(pkg, prob, rank, world):
    """This rank's share of the FIXED problem `prob` split `world` ways by (batch x head):
    views of its slices (contiguous in [B,H,S,D]), the work they hold and the launch."""
    q, k, v = prob.inputs
    B, H, S, D = q.shape
    b, e = pkg.sharding.attention_shard(B, H, rank, world)
    flat = [t.view(1, B * H, S, D)[:, b:e] for t in (q, k, v)]
    out = prob.out.view(1, B * H, S, D)[:, b:e]
    return flat, out, prob.work * (e - b) / (B * H), e - b


def gemm_problem(ops, dev, name, rank):
    import torch
    M, N, K, seed = GEMM_WORKLOADS[name]
    g = torch.Generator(device=dev).manual_seed(seed)
    a = (torch.rand(M, K, device=dev, generator=g) * 2 - 1).to(torch.bfloat16)
    g.manual_seed(seed + 1 + rank)
    bt = (torch.rand(N, K, device=dev, generator=g) * 2 - 1).to(torch.bfloat16)
    o = torch.empty(M, N, device=dev, dtype=torch.bfloat16)

    def run(ins, out, stream=None):
        ops.gemm(ins[0], ins[1], out=out, stream=stream)

    return Problem(name, [a, bt], o, run, 2.0 * M * N * K, (M * K + N * K + M * N) * 2,
                   f"{name}: M={M} N={N} K={K} bf16 out")


def rowwise_problem(ops, dev, name, rank, rows_override):
    import torch
    rows, N, seed = ROWWISE_WORKLOADS[name]
    rows = rows_override or rows
    g = torch.Generator(device=dev).manual_seed(seed + rank)
    x = torch.randn(rows, N, device=dev, generator=g)
    w = torch.randn(N, device=dev, generator=g) * 0.1 + 1.0
    bias = torch.randn(N, device=dev, generator=g) * 0.1
    inputs = [x, torch.randn(rows, N, device=dev, generator=g)] if name == "swiglu" else [x]

    def run(ins, out, stream=None):
        if name == "softmax":
            ops.softmax(ins[0], out=out, stream=stream)
        elif name == "rms_norm":
            ops.rms_norm(ins[0], w, 1e-6, out=out, stream=stream)
        elif name == "layer_norm":
            ops.layer_norm(ins[0], w, bias, 1e-5, out=out, stream=stream)
        else:
            ops.swiglu(ins[0], ins[1], out=out, stream=stream)

    nbytes = (len(inputs) + 1) * rows * N * 4
    return Problem(name, inputs, torch.empty_like(x), run, float(nbytes), nbytes, f"{name}: rows={rows} N={N} fp32")


class Bench:
    """Timing discipline shared by every measurement of the native arm: a time-based
    warm-up (the reference spins launches for 25 ms before it times, bench/flash_attention.jl:
    113-127), then `repeats` regions of exactly `steps` back-to-back launches, each bracketed
    by barrier + synchronize and timed with CUDA events on the launching stream; a region's
    time is the max over ranks, the reported figure the median over regions."""

    def __init__(self, torch, dist, world, dev, sampler):
        self.torch, self.dist, self.world, self.dev, self.sampler = torch, dist, world, dev, sampler

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, x):
        t = self.torch.tensor([x], dtype=self.torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t[0])

    warm_ms = 25.0

    def warm(self, launch, min_launches, min_ms=None):
        min_ms = self.warm_ms if min_ms is None else min_ms
        launch()                          # the first call pays one-time set-up (module load,
        self.torch.cuda.synchronize()     # attributes, scratch): keep it out of the warm-up clock
        t0, n = time.perf_counter(), 1
        while n < max(min_launches, 3) or (time.perf_counter() - t0) * 1e3 < min_ms:
            launch()
            n += 1
            if n % 8 == 0:
                self.torch.cuda.synchronize()   # keep the queue short so the wall clock means something
        self.torch.cuda.synchronize()
        return n

    def region(self, launch, steps):
        """One timed region of exactly `steps` launches: (ms max over ranks, clocks seen)."""
        torch = self.torch
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for _ in range(steps):
            launch()
        e1.record()
        self.barrier()
        t1 = time.perf_counter()
        return self.max_over_ranks(e0.elapsed_time(e1)), self.sampler.window(t0, t1)

    def measure(self, launch, steps, warmup, repeats=5):
        n_warm = self.warm(launch, warmup)
        regions = [self.region(launch, steps) for _ in range(repeats)]
        ms = sorted(r[0] / steps for r in regions)
        mid = regions[sorted(range(repeats), key=lambda i: regions[i][0])[repeats // 2]]
        return {"ms": ms[repeats // 2], "ms_min": ms[0], "ms_max": ms[-1], "repeats": repeats, "steps": steps,
                "warmup_launches": n_warm, "clocks": mid[1]}


def quantisation_note(pkg, name, world, sm):
    """What the item count alone allows at `world` ranks (a bound, not a measurement)."""
    if name in GEMM_WORKLOADS:
        M, N, K, _ = GEMM_WORKLOADS[name]
        tiles = (M // 256) * ((N // world) // 256)
        waves = tiles / (sm // 2)
        return f"{tiles} tiles of 256x256 on {sm // 2} SM pairs = {waves:.2f} waves: at most {waves / math.ceil(waves):.2f} of linear"
    B, H, S, D, causal, _, _ = WORKLOADS[name]
    items = (B * H // world) * ((S + 255) // 256)
    waves = items / sm
    return (f"{items} items of 256 rows on {sm} SMs = {waves:.2f} rounds: whole items allow "
            f"{waves / math.ceil(waves):.2f} of linear (the last round is cut along the key axis only where that "
            f"is expected to pay)")


def run_native_arm(args):
    # stdout carries exactly one line, the JSON record: libraries that write to file
    # descriptor 1 (NCCL prints its version there when a communicator is created) are
    # sent to stderr for the duration of the run
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    import torch
    import torch.distributed as dist
    import __graft_entry__ as ge

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    local_cpus = None
    if world > 1:
        pr = torch.cuda.get_device_properties(local_rank)
        bus = (f"{pr.pci_domain_id:08x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
               if hasattr(pr, "pci_bus_id") else None)
        local_cpus = bind_to_gpu_local_cpus(physical_gpu_index(local_rank), bus)
        dist.init_process_group("nccl", device_id=dev)
    pkg = ge.load_package()
    ops = pkg.ops
    pkg.native.lib()   # fail loudly here if the CUDA library is missing
    sm_count = torch.cuda.get_device_properties(local_rank).multi_processor_count
    peak_burst, peak_sustained, peak_hbm, peak_kind = peaks()

    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    bench = Bench(torch, dist, world, dev, sampler)
    bench.warm_ms = args.warm_ms

    def check_status(where):
        status = ops.sync_status()
        if status != 0:
            raise SystemExit(f"device status after {where}: " + pkg.native.strerror(status))

    # ---- the headline workload: one full configuration per rank ("weak") ----
    unit, unit_scale, bound = "TFLOPS", 1e12, "tensor"
    if args.workload in ROWWISE_WORKLOADS:
        prob = rowwise_problem(ops, dev, args.workload, rank, args.rows)
        unit, unit_scale, bound = "GB/s", 1e9, "hbm"
        metric = f"{args.workload} GB/s (fp32 in, fp32 out, algorithmic bytes), {prob.text} per GPU"
        shard_text = "sharded by rows"
    elif args.workload in GEMM_WORKLOADS:
        prob = gemm_problem(ops, dev, args.workload, rank)
        metric = "GEMM TFLOPS (bf16 in, fp32 accumulate, bf16 out), M=N=K=8192 per GPU"
        shard_text = "C split by column blocks, A replicated"
    else:
        prob = attention_problem(ops, dev, args.workload, seed_offset=rank)
        metric = METRIC if args.workload == "c2" else f"attention fwd TFLOPS (bf16, fp32 accumulate), {args.workload}"
        shard_text = f"sharded by batch*head, global batch {WORKLOADS[args.workload][0] * world}"
    seed = (WORKLOADS.get(args.workload) or GEMM_WORKLOADS.get(args.workload) or ROWWISE_WORKLOADS[args.workload])[-1]

    head = bench.measure(lambda: prob.run(prob.inputs, prob.out), args.steps, args.warmup)
    check_status("the headline region")
    ms_per_step = head["ms"]
    value = prob.work * world / (ms_per_step * 1e-3) / unit_scale
    achieved = prob.work / (ms_per_step * 1e-3) / unit_scale   # one launch on one GPU
    # launches run back to back from the warm-up to the last region: a quarter of a second of
    # that puts the GPU under its power cap, where the sustained cuBLAS figure is the fair peak
    busy_ms = ms_per_step * (head["warmup_launches"] + head["steps"] * head["repeats"])
    if bound == "tensor":
        long_run = busy_ms >= 250.0
        peak = peak_sustained if long_run else peak_burst
        peak_text = f"{peak_kind} ({'sustained' if long_run else 'burst'} cuBLAS bf16)"
    else:
        peak, peak_text = peak_hbm, f"{peak_kind} (copy)"

    # ---- the other configurations, one burst each, and the fixed problems split over the ranks ----
    configs, strong, problems = {}, {}, {}
    extra = args.workload == "c2" and not args.headline_only
    head_mhz = head["clocks"]["sm_mhz"]
    if extra:
        # one burst of each other configuration, right behind the headline (same, cool state)
        problems["c2"] = prob
        for name in ("c3", "c4", "c5"):
            is_gemm = name in GEMM_WORKLOADS
            steps_n = {"c4": 5}.get(name, 20)
            full = gemm_problem(ops, dev, name, 0) if is_gemm else attention_problem(ops, dev, name)
            problems[name] = full
            full_t = bench.measure(lambda: full.run(full.inputs, full.out), steps_n, 3, repeats=3)
            check_status(f"configs.{name}")
            tf = full.work / (full_t["ms"] * 1e-3) / 1e12
            configs[name] = {"workload": full.text, "ms": full_t["ms"], "ms_min": full_t["ms_min"],
                             "ms_max": full_t["ms_max"], "tflops": tf, "frac_of_burst_peak": tf / peak_burst,
                             "frac_of_sustained_peak": tf / peak_sustained,
                             "steps": steps_n, "repeats": 3, "sm_mhz": full_t["clocks"]["sm_mhz"],
                             "kcycles_per_launch": (full_t["ms"] * full_t["clocks"]["sm_mhz"]
                                                    if full_t["clocks"]["sm_mhz"] else None)}
            configs[name]["power_w"] = full_t["clocks"].get("power_w")
            if is_gemm:
                # the vendor library on the same operands, same box, same moment: what the measured
                # peak looks like today (library code: measured beside the product, never on its path)
                a_op, bt_op = full.inputs
                lib_out = torch.empty_like(full.out)
                lib_t = bench.measure(lambda: torch.matmul(a_op, bt_op.t(), out=lib_out), steps_n, 3, repeats=3)
                configs[name]["cublas_same_run"] = {
                    "ms": lib_t["ms"], "tflops": full.work / (lib_t["ms"] * 1e-3) / 1e12,
                    "sm_mhz": lib_t["clocks"]["sm_mhz"], "power_w": lib_t["clocks"].get("power_w")}
                del lib_out
            if name == "c3":
                # at D = 64 the exponentials, not the tensor pipe, bound a tile: 16 ex2/clk/SM on the
                # MUFU (measured: profiles/ex2_throughput.md) against 2*D flop per score on the tensor pipe
                configs[name]["mufu_ceiling_tflops"] = 4.0 * 64 * 16 * sm_count * (full_t["clocks"]["sm_mhz"] or 0) * 1e6 / 1e12

    # ---- sustained: one region of at least half a second (power management settles) ----
    sustained = None
    if bound == "tensor" and not args.headline_only:
        n_long = max(args.steps, int(math.ceil(600.0 / ms_per_step)))
        ms_long, clk_long = bench.region(lambda: prob.run(prob.inputs, prob.out), n_long)
        check_status("the sustained region")
        tf_long = prob.work / (ms_long / n_long * 1e-3) / 1e12
        mhz = clk_long["sm_mhz"]
        sustained = {"launches": n_long, "region_ms": ms_long, "ms_per_step": ms_long / n_long,
                     "tflops_per_gpu": tf_long, "peak": peak_sustained,
                     "frac": tf_long / peak_sustained, "peak_kind": f"{peak_kind} (sustained cuBLAS bf16)",
                     "clocks": clk_long,
                     "kcycles_per_launch": (ms_long / n_long) * mhz if mhz else None}

    if extra:
        # the fixed problems split over the ranks ("strong"), after the long region: steady clocks
        for name in ("c2", "c3", "c4", "c5"):
            is_gemm = name in GEMM_WORKLOADS
            steps_n = {"c4": 5}.get(name, 20)
            full = problems[name]

            def shard_launcher(n_ranks, r):
                # a shard writes to a buffer of its own: the resident output of the headline run stays
                # what the end-to-end leg is compared with
                if is_gemm:
                    a, bt = full.inputs
                    b, e = pkg.sharding.gemm_column_shard(bt.shape[0], r, n_ranks)
                    bt_s = bt[b:e]
                    out = torch.empty(a.shape[0], e - b, device=dev, dtype=torch.bfloat16)
                    return (lambda: full.run([a, bt_s], out)), f"{e - b} of {bt.shape[0]} columns"
                ins, out_view, _, n_sl = attention_shard(pkg, full, r, n_ranks)
                out = torch.empty_like(out_view)
                return (lambda: full.run(ins, out)), f"{n_sl} of {full.inputs[0].shape[0] * full.inputs[0].shape[1]} (batch, head) slices"

            def timed(launch):
                # regions of at least 25 ms each, so that both sides of a ratio sit in the same power
                # state and the clock sampler sees each region
                probe = bench.measure(launch, 5, 3, repeats=1)["ms"]
                n = int(bench.max_over_ranks(max(steps_n, math.ceil(25.0 / max(probe, 1e-3)))))
                t = bench.measure(launch, n, 3, repeats=3)
                mhz = t["clocks"]["sm_mhz"]
                return t["ms"], (t["ms"] * mhz if mhz else None)

            # the whole problem is timed again right before and right after its shards, so that
            # both sides of the ratio see the same clocks (the headline above ran on a cooler GPU)
            full_launch = lambda: full.run(full.inputs, full.out)
            f0_ms, f0_kc = timed(full_launch)
            entry = {"workload": full.text}
            if world > 1:
                launch, what = shard_launcher(world, rank)
                sh_ms, sh_kc = timed(launch)
                shards = {str(world): (what, sh_ms, sh_kc)}
            else:
                # one GPU: the shards a rank would hold at 2, 4 and 8 ranks, timed one after the
                # other (ranks are independent: no collective on the path)
                shards = {}
                for n_ranks in (2, 4, 8):
                    launch, what = shard_launcher(n_ranks, 0)
                    sh_ms, sh_kc = timed(launch)
                    shards[str(n_ranks)] = (what, sh_ms, sh_kc)
            f1_ms, f1_kc = timed(full_launch)
            check_status(f"strong.{name}")
            t1_ms = 0.5 * (f0_ms + f1_ms)
            t1_kc = 0.5 * (f0_kc + f1_kc) if (f0_kc and f1_kc) else None
            entry["t1_ms"] = t1_ms
            entry["t1_kcycles"] = t1_kc

            def eff(n_ranks, sh_ms, sh_kc):
                return {"ms": sh_ms, "tflops_total": full.work / (sh_ms * 1e-3) / 1e12,
                        "efficiency": t1_ms / (n_ranks * sh_ms),
                        "efficiency_in_cycles": (t1_kc / (n_ranks * sh_kc)) if (t1_kc and sh_kc) else None,
                        "bound": quantisation_note(pkg, name, n_ranks, sm_count)}

            if world > 1:
                what, sh_ms, sh_kc = shards[str(world)]
                entry.update({"n": world, "shard_per_rank": what, **eff(world, sh_ms, sh_kc)})
            else:
                entry.update({"n": 1, "efficiency": 1.0,
                              "single_gpu_emulation": {k: {"shard": v[0], **eff(int(k), v[1], v[2])}
                                                       for k, v in shards.items()}})
            strong[name] = entry
        problems.clear()
        torch.cuda.empty_cache()

    # ---- end to end: host buffers in, host buffer out, copies inside the timed region ----
    inputs, o = prob.inputs, prob.out
    e2e_steps = max(3, min(args.steps, 10))
    nbuf = 3

    def e2e_measure(ins, want):
        """`e2e_steps` steps of: pinned host inputs -> device, the launch, device output ->
        pinned host; three streams and `nbuf` buffer sets, so the copy-in of the next steps and
        the copy-out of the previous one overlap the kernel of step i. Returns (ms per step, max
        over ranks; whether the last host output equals `want`, the resident run's output)."""
        h_in = [[torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in ins] for _ in range(nbuf)]
        h_out = [torch.empty(want.shape, dtype=want.dtype).pin_memory() for _ in range(nbuf)]
        for b in range(nbuf):
            for h, t in zip(h_in[b], ins):
                h.copy_(t)
        d_in = [[torch.empty_like(t) for t in ins] for _ in range(nbuf)]
        d_out = [torch.empty_like(want) for _ in range(nbuf)]
        s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        ev_in = [torch.cuda.Event() for _ in range(nbuf)]
        ev_cmp = [torch.cuda.Event() for _ in range(nbuf)]
        ev_out = [torch.cuda.Event() for _ in range(nbuf)]

        def loop(n):
            for i in range(n):
                b = i % nbuf
                with torch.cuda.stream(s_in):
                    s_in.wait_event(ev_cmp[b])          # device inputs of slot b no longer in use
                    for d, h in zip(d_in[b], h_in[b]):
                        d.copy_(h, non_blocking=True)
                    ev_in[b].record(s_in)
                with torch.cuda.stream(s_cmp):
                    s_cmp.wait_event(ev_in[b])
                    s_cmp.wait_event(ev_out[b])         # device output of slot b already copied out
                    prob.run(d_in[b], d_out[b], stream=s_cmp)
                    ev_cmp[b].record(s_cmp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_cmp[b])
                    h_out[b].copy_(d_out[b], non_blocking=True)
                    ev_out[b].record(s_out)

        loop(nbuf)
        bench.barrier()
        t0 = time.perf_counter()
        loop(e2e_steps)
        torch.cuda.synchronize()
        ms_local = (time.perf_counter() - t0) * 1e3
        ms_step = bench.max_over_ranks(ms_local) / e2e_steps
        same = bool(torch.equal(h_out[(e2e_steps - 1) % nbuf].to(dev), want))
        return ms_step, same

    def nbytes(ts):
        return sum(t.numel() * t.element_size() for t in ts)

    e2e_ms_step, e2e_ok = e2e_measure(inputs, o)
    e2e_value = prob.work * world / (e2e_ms_step * 1e-3) / unit_scale
    h2d_bytes = nbytes(inputs)
    d2h_bytes = nbytes([o])
    check_status("the end-to-end region")

    # the same call with K and V shared by groups of four query heads (the entry point's
    # grouped-head form): the same flops from half the bytes over PCIe
    e2e_grouped = None
    if args.workload in WORKLOADS and not args.headline_only:
        q, k, v = inputs
        group = 4
        kg, vg = (t[:, : t.shape[1] // group].contiguous() for t in (k, v))
        o_g = torch.empty_like(o)
        prob.run([q, kg, vg], o_g)
        torch.cuda.synchronize()
        g_ms, g_ok = e2e_measure([q, kg, vg], o_g)
        check_status("the grouped-head end-to-end region")
        g_h2d = nbytes([q, kg, vg])
        e2e_grouped = {"kv_heads": int(kg.shape[1]), "query_heads": int(q.shape[1]),
                       "value": prob.work * world / (g_ms * 1e-3) / unit_scale, "unit": unit,
                       "ms_per_step": g_ms, "h2d_bytes_per_step": g_h2d, "d2h_bytes_per_step": d2h_bytes,
                       "h2d_gbs_per_rank": g_h2d / (g_ms * 1e-3) / 1e9, "matches_resident_run": g_ok}
        del kg, vg, o_g

    # verification checksum gathered over ranks (outside every timed region)
    cs = torch.tensor([float(o.float().sum()), float(o.float().abs().sum())], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(cs)
    sampler.stop()

    if rank == 0:
        line = {
            "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "warmup_launches": head["warmup_launches"], "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if bound == "tensor" else "f32", "data": "synthetic",
            "config": {"workload": f"{prob.text} per GPU, {shard_text}",
                       "l2": f"inputs+output {prob.algo_bytes >> 20} MiB per launch > 126 MB L2, no explicit flush",
                       "seed": seed, "parallelism": f"dp{world} (independent shards, no collective)",
                       "timing": f"warm-up >= 25 ms and >= {max(args.warmup, 3)} launches, then {head['repeats']} regions of "
                                 f"{args.steps} launches; value = median region, max over ranks"},
            "per_gpu_tflops" if bound == "tensor" else "per_gpu_gbs": value / world,
            "ms_per_step_min": head["ms_min"], "ms_per_step_max": head["ms_max"], "repeats": head["repeats"],
            "roofline": {"bound": bound, "achieved": achieved, "peak": peak,
                         "unit": "TFLOP/s" if bound == "tensor" else "GB/s",
                         "frac": achieved / peak, "traffic": None if args.rows else NCU_TRAFFIC_BYTES.get(args.workload),
                         "peak_kind": peak_text,
                         "algorithmic_flops_per_launch": prob.work if bound == "tensor" else None,
                         "algorithmic_bytes_per_launch": prob.algo_bytes,
                         "kcycles_per_launch": ms_per_step * head_mhz if head_mhz else None},
            "e2e": {"value": e2e_value, "unit": unit, "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": d2h_bytes, "ms_per_step": e2e_ms_step, "steps": e2e_steps,
                    "h2d_gbs_per_rank": h2d_bytes / (e2e_ms_step * 1e-3) / 1e9,
                    "h2d_gbs_all_ranks": world * h2d_bytes / (e2e_ms_step * 1e-3) / 1e9,
                    "buffer_sets": nbuf,
                    "d2h_gbs_per_rank": d2h_bytes / (e2e_ms_step * 1e-3) / 1e9,
                    "matches_resident_run": e2e_ok, "rank0_gpu_local_cpus": local_cpus},
            "gpu_launches": args.steps,
            "clocks": head["clocks"],
            "checksum": {"sum": float(cs[0]), "abs_sum": float(cs[1])},
        }
        if e2e_grouped is not None:
            line["e2e"]["grouped_kv"] = e2e_grouped
        if sustained is not None:
            line["sustained"] = sustained
        if configs:
            line["configs"] = configs
        if strong:
            line["strong"] = strong
        if world == 1 and not args.no_cpu_baseline and args.workload in WORKLOADS:
            # the CPU oracle on the first slices of THIS run's inputs: timed as the CPU
            # baseline, and its output is the spot check of what the GPU wrote
            import numpy as np
            import oracle
            oracle.build_c_oracle()
            B, H, S, D, causal, _, _ = WORKLOADS[args.workload]
            n_slices = 16
            hb = [t.view(B * H, S, D)[:n_slices].cpu().view(torch.int16).numpy().view(np.uint16) for t in inputs]
            t0 = time.perf_counter()
            ref = oracle.attention_ref_c(hb[0], hb[1], hb[2], 1.0 / math.sqrt(D), causal, nthreads=host_threads())
            cpu_s = time.perf_counter() - t0
            err = np.abs(o.view(B * H, S, D)[:n_slices].float().cpu().numpy() - ref)
            line["cpu_baseline"] = {"value": attn_flops(1, n_slices, S, D, causal) / cpu_s / 1e12, "unit": "TFLOPS",
                                    "cores": host_threads(), "kind": "port",
                                    "sample": f"{n_slices} of {B * H} (batch, head) slices of the workload, "
                                              f"{cpu_s:.2f} s wall"}
            line["oracle_check"] = {"slices": n_slices, "max_abs_err": float(err.max()), "mean_abs_err": float(err.mean()),
                                    "ok": bool(err.max() <= 2e-2 and err.mean() <= 2e-3)}
        if world == 1 and not args.no_cpu_baseline and args.workload in ROWWISE_WORKLOADS:
            rows = ROWWISE_WORKLOADS[args.workload][0]
            cpu_gbs, cpu_s = rowwise_cpu_sample(args.workload, 16384)
            line["cpu_baseline"] = {"value": cpu_gbs, "unit": "GB/s", "cores": 1, "kind": "port",
                                    "sample": f"16384 of {rows} rows of the workload, numpy float64, {cpu_s:.2f} s wall"}
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["native", "reference"], default="native")
    ap.add_argument("--workload", choices=sorted(WORKLOADS) + sorted(GEMM_WORKLOADS) + sorted(ROWWISE_WORKLOADS),
                    default="c2")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--headline-only", action="store_true",
                    help="skip the `sustained`, `configs` and `strong` blocks (the long region, the other "
                         "configurations and the fixed problems split over the ranks): for profiler captures")
    ap.add_argument("--warm-ms", type=float, default=25.0,
                    help="minimum wall time of every warm-up (0 under a profiler, where each launch is replayed)")
    ap.add_argument("--rows", type=int, default=0,
                    help="row-wise workloads only: rows per GPU instead of the default (for small profiler captures)")
    args = ap.parse_args()
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        # launched without torchrun: start one process per GPU ourselves
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(29400 + os.getpid() % 500),
               os.path.abspath(__file__)] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_native_arm(args)


if __name__ == "__main__":
    main()
