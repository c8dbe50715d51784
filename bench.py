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
copies of Q, K, V and the device -> host copy of O inside the timed region.
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
NCU_TRAFFIC_BYTES = {"c2": 201.44e6 + 43.03e6, "c3": 201.38e6 + 45.59e6, "c4": 1649.54e6 + 517.57e6,
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


def measured_peak(region_ms):
    """bf16 tensor peak to divide by: the pool's measured cuBLAS figure (burst for a
    short timed region, sustained for one long enough to sit under the power cap)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            mp = json.load(f)
        if region_ms >= 500.0 and "bf16_tflops_sustained" in mp:
            return float(mp["bf16_tflops_sustained"]), "measured (sustained cuBLAS bf16)"
        return float(mp["bf16_tflops"]), "measured (burst cuBLAS bf16)"
    except Exception:
        return FALLBACK_PEAK_TFLOPS, "fallback"


def measured_hbm_peak():
    """HBM copy bandwidth to divide by (GB/s): the pool's measured STREAM-style copy."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (copy)"
    except Exception:
        return FALLBACK_PEAK_GBS, "fallback"


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
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop_evt = threading.Event()
        self.active = False

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {
                "hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown,
                "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown,
                "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap,
            }
            while not self._stop_evt.is_set():
                if self.active:
                    self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                    for k, bit in names.items():
                        if r & bit:
                            self.reasons.add(k)
                time.sleep(0.002)
        except Exception as e:  # NVML missing: report that instead of inventing numbers
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")

    def stop(self):
        self._stop_evt.set()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "samples": len(self.samples), "reasons": sorted(self.reasons)}


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
def cpu_sample(workload, n_slices, repeats=1):
    """Times the CPU oracle (C port of the reference's fab_cpu_ref) on `n_slices`
    (batch, head) slices of the workload with every host thread. Returns TFLOPS."""
    import numpy as np
    import oracle
    oracle.build_c_oracle()
    B, H, S, D, causal, sigma, seed = WORKLOADS[workload]
    rng = np.random.default_rng(seed)
    q, k, v = (oracle.to_bf16_bits((rng.standard_normal((n_slices, S, D)) * s).astype(np.float32))
               for s in (sigma, sigma, 1.0))
    best = float("inf")
    for _ in range(repeats):
        t = time.perf_counter()
        oracle.attention_ref_c(q, k, v, 1.0 / math.sqrt(D), causal, nthreads=host_threads())
        best = min(best, time.perf_counter() - t)
    return attn_flops(1, n_slices, S, D, causal) / best / 1e12, best, host_threads()


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
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pkg = ge.load_package()
    ops = pkg.ops
    pkg.native.lib()   # fail loudly here if the CUDA library is missing

    unit, unit_scale, bound = "TFLOPS", 1e12, "tensor"
    if args.workload in ROWWISE_WORKLOADS:
        # this rank's block of rows (world * rows in all): independent rows, no collective
        rows, N, seed = ROWWISE_WORKLOADS[args.workload]
        rows = args.rows or rows
        g = torch.Generator(device=dev).manual_seed(seed + rank)
        x = torch.randn(rows, N, device=dev, generator=g)
        w = torch.randn(N, device=dev, generator=g) * 0.1 + 1.0
        bias = torch.randn(N, device=dev, generator=g) * 0.1
        o = torch.empty_like(x)
        if args.workload == "swiglu":
            inputs = [x, torch.randn(rows, N, device=dev, generator=g)]
        else:
            inputs = [x]
        algo_bytes = (len(inputs) + 1) * rows * N * 4
        flops_rank = float(algo_bytes)   # the unit of work of this family is the algorithmic byte
        unit, unit_scale, bound = "GB/s", 1e9, "hbm"
        metric = f"{args.workload} GB/s (fp32 in, fp32 out, algorithmic bytes), rows={rows} N={N} per GPU"
        wl_text = f"{args.workload}: rows={rows} N={N} fp32 per GPU, sharded by rows"
        l2_text = f"input+output {algo_bytes >> 20} MiB per launch > 126 MB L2, no explicit flush"
        rw_name = args.workload

        def run(ins, out, stream=None):
            if rw_name == "softmax":
                ops.softmax(ins[0], out=out, stream=stream)
            elif rw_name == "rms_norm":
                ops.rms_norm(ins[0], w, 1e-6, out=out, stream=stream)
            elif rw_name == "layer_norm":
                ops.layer_norm(ins[0], w, bias, 1e-5, out=out, stream=stream)
            else:
                ops.swiglu(ins[0], ins[1], out=out, stream=stream)
    elif args.workload in GEMM_WORKLOADS:
        # C[M, N*world] = A[M,K] B[K, N*world]: A replicated, this rank owns one block of N columns
        M, N, K, seed = GEMM_WORKLOADS[args.workload]
        g = torch.Generator(device=dev).manual_seed(seed)
        a = (torch.rand(M, K, device=dev, generator=g) * 2 - 1).to(torch.bfloat16)
        g.manual_seed(seed + 1 + rank)
        bt = (torch.rand(N, K, device=dev, generator=g) * 2 - 1).to(torch.bfloat16)
        o = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        inputs = [a, bt]
        flops_rank = 2.0 * M * N * K
        algo_bytes = (M * K + N * K + M * N) * 2
        metric = "GEMM TFLOPS (bf16 in, fp32 accumulate, bf16 out), M=N=K=8192 per GPU"
        wl_text = f"{args.workload}: M={M} N={N} K={K} per GPU, C split by column blocks, A replicated"
        l2_text = "A+B+C 384 MiB per launch > 126 MB L2, no explicit flush"

        def run(ins, out, stream=None):
            ops.gemm(ins[0], ins[1], out=out, stream=stream)
    else:
        B, H, S, D, causal, sigma, seed = WORKLOADS[args.workload]
        # this rank's shard of the global batch (world * B): B x H slices, generated locally
        g = torch.Generator(device=dev).manual_seed(seed + rank)
        q = (torch.randn(B, H, S, D, device=dev, generator=g) * sigma).to(torch.bfloat16)
        k = (torch.randn(B, H, S, D, device=dev, generator=g) * sigma).to(torch.bfloat16)
        v = torch.randn(B, H, S, D, device=dev, generator=g).to(torch.bfloat16)
        o = torch.empty_like(q)
        inputs = [q, k, v]
        sm_scale = 1.0 / math.sqrt(D)
        flops_rank = attn_flops(B, H, S, D, causal)
        algo_bytes = 4 * q.numel() * 2
        metric = METRIC if args.workload == "c2" else f"attention fwd TFLOPS (bf16, fp32 accumulate), {args.workload}"
        wl_text = (f"{args.workload}: B={B} H={H} S={S} D={D} causal={causal} per GPU, sharded by batch*head, "
                   f"global batch {B * world}")
        l2_text = f"inputs+output {4 * q.numel() * 2 >> 20} MiB per launch > 126 MB L2, no explicit flush"

        def run(ins, out, stream=None):
            ops.fa_fwd(ins[0], ins[1], ins[2], causal=causal, sm_scale=sm_scale, out=out, stream=stream)

    def step():
        run(inputs, o)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.active = True
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    sampler.active = False
    status = ops.sync_status()
    if status != 0:
        raise SystemExit("device status: " + pkg.native.strerror(status))
    region_ms = e0.elapsed_time(e1)
    t = torch.tensor([region_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    region_ms_max = float(t[0])
    ms_per_step = region_ms_max / args.steps
    value = flops_rank * world / (ms_per_step * 1e-3) / unit_scale

    # ---- end to end: host buffers in, host buffer out, copies inside the timed region ----
    e2e_steps = max(3, min(args.steps, 10))
    nbuf = 2
    h_in = [[torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in inputs] for _ in range(nbuf)]
    h_out = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for _ in range(nbuf)]
    for b in range(nbuf):
        for h, t in zip(h_in[b], inputs):
            h.copy_(t)
    d_in = [[torch.empty_like(t) for t in inputs] for _ in range(nbuf)]
    d_out = [torch.empty_like(o) for _ in range(nbuf)]
    s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(nbuf)]
    ev_cmp = [torch.cuda.Event() for _ in range(nbuf)]
    ev_out = [torch.cuda.Event() for _ in range(nbuf)]

    def e2e_loop(n):
        # three streams, two buffer sets: the copy-in of step i+1 and the copy-out of
        # step i-1 overlap the kernel of step i
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
                run(d_in[b], d_out[b], stream=s_cmp)
                ev_cmp[b].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp[b])
                h_out[b].copy_(d_out[b], non_blocking=True)
                ev_out[b].record(s_out)

    e2e_loop(2)
    barrier()
    t0 = time.perf_counter()
    e2e_loop(e2e_steps)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    t = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms_step = float(t[0]) / e2e_steps
    e2e_value = flops_rank * world / (e2e_ms_step * 1e-3) / unit_scale
    e2e_ok = bool(torch.equal(h_out[(e2e_steps - 1) % nbuf].to(dev), o))
    h2d_bytes = sum(t.numel() * t.element_size() for t in inputs)
    d2h_bytes = o.numel() * o.element_size()
    sampler.stop()
    status = ops.sync_status()
    if status != 0:
        raise SystemExit("device status: " + pkg.native.strerror(status))

    # verification checksum gathered over ranks (outside every timed region)
    cs = torch.tensor([float(o.float().sum()), float(o.float().abs().sum())], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(cs)

    if rank == 0:
        peak, peak_kind = measured_peak(region_ms_max) if bound == "tensor" else measured_hbm_peak()
        achieved = flops_rank / (ms_per_step * 1e-3) / unit_scale   # one launch on one GPU
        line = {
            "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if bound == "tensor" else "f32", "data": "synthetic",
            "config": {"workload": wl_text, "l2": l2_text,
                       "seed": seed, "parallelism": f"dp{world} (independent shards, no collective)"},
            "per_gpu_tflops" if bound == "tensor" else "per_gpu_gbs": value / world,
            "roofline": {"bound": bound, "achieved": achieved, "peak": peak,
                         "unit": "TFLOP/s" if bound == "tensor" else "GB/s",
                         "frac": achieved / peak, "traffic": None if args.rows else NCU_TRAFFIC_BYTES.get(args.workload),
                         "peak_kind": peak_kind,
                         "algorithmic_flops_per_launch": flops_rank if bound == "tensor" else None,
                         "algorithmic_bytes_per_launch": algo_bytes},
            "e2e": {"value": e2e_value, "unit": unit, "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": d2h_bytes, "ms_per_step": e2e_ms_step, "steps": e2e_steps,
                    "matches_resident_run": e2e_ok, "rank0_gpu_local_cpus": local_cpus},
            "gpu_launches": args.steps,
            "clocks": sampler.summary(),
            "checksum": {"sum": float(cs[0]), "abs_sum": float(cs[1])},
        }
        if world == 1 and not args.no_cpu_baseline and args.workload in WORKLOADS:
            n_slices = 16
            cpu_tf, cpu_s, threads = cpu_sample(args.workload, n_slices)
            line["cpu_baseline"] = {"value": cpu_tf, "unit": "TFLOPS", "cores": threads, "kind": "port",
                                    "sample": f"{n_slices} of {B * H} (batch, head) slices of the workload, "
                                              f"{cpu_s:.2f} s wall"}
        if world == 1 and not args.no_cpu_baseline and args.workload in ROWWISE_WORKLOADS:
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
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["native", "reference"], default="native")
    ap.add_argument("--workload", choices=sorted(WORKLOADS) + sorted(GEMM_WORKLOADS) + sorted(ROWWISE_WORKLOADS),
                    default="c2")
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
