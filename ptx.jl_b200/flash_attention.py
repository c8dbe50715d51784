"""Host-side mirror of the reference's attention workbench entry points.

Same names, arguments and return shape as bench/flash_attention.jl --
fab_setup(B, H, S; input_scale, cfg) -> (launch!, O_d, dbg_d, Q, K, V, sm_scale,
B, H, S, num_ctas, keepalive)  (:41-85), fab_check (:89-105), fab_time (:109-136),
fab_sweep (:140-158), fab_hang_debug (:163-179) -- with the launch closure calling
the native fa_fwd_bf16 instead of a Julia-compiled kernel. Differences, all
additive: head dim 64 and a causal flag are accepted; `cfg` carries the native
flags instead of the DSL kernel's compile-time knobs.

The checker is passed in by the caller (tests hand over the CPU oracle); this
module never computes attention on the host.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, Optional

import torch

from . import native, ops

FAB_BM = 128          # rows per Q sub-tile (flash_attention_defs.jl:124)
FAB_QSTAGE = 2        # sub-tiles per work item (:125)
FAB_BN = 128          # KV tile (:126)
FAB_CFG_DEFAULT: Dict[str, object] = {"flags": 0, "causal": False, "head_dim": 128}


@dataclass
class FabProblem:
    """What fab_setup returns (bench/flash_attention.jl:83-85)."""
    launch: Callable[[], None]
    O_d: torch.Tensor
    dbg_d: torch.Tensor
    Q: torch.Tensor          # host fp32, (B*H*S, D)
    K: torch.Tensor
    V: torch.Tensor
    sm_scale: float
    B: int
    H: int
    S: int
    D: int
    causal: bool
    num_ctas: int
    keepalive: tuple = field(default_factory=tuple)


def fab_pack(x: torch.Tensor) -> torch.Tensor:
    """fp32 (rows, D) -> bf16, row-major (flash_attention_defs.jl:979-986)."""
    return x.to(torch.bfloat16).contiguous()


def fab_setup(B: int, H: int, S: int, *, input_scale: float = 0.5,
              cfg: Optional[Dict[str, object]] = None, device: Optional[torch.device] = None) -> FabProblem:
    cfg = {**FAB_CFG_DEFAULT, **(cfg or {})}
    D = int(cfg["head_dim"])
    causal = bool(cfg["causal"])
    if S % (FAB_QSTAGE * FAB_BM) != 0:
        raise ValueError("S must be a multiple of 256 (bench/flash_attention.jl:43)")
    device = device or torch.device("cuda", torch.cuda.current_device())
    total_rows = B * H * S
    total_work = (S // (FAB_QSTAGE * FAB_BM)) * B * H
    n_sms = torch.cuda.get_device_properties(device).multi_processor_count
    sm_scale = 1.0 / math.sqrt(D)
    # Seed formula of the reference (:56); the stream itself is torch's, not Julia's.
    gen = torch.Generator().manual_seed(B * 7919 + H * 131 + S)
    Q = torch.randn(total_rows, D, generator=gen) * input_scale
    K = torch.randn(total_rows, D, generator=gen) * input_scale
    V = torch.randn(total_rows, D, generator=gen)
    Q_d, K_d, V_d = (fab_pack(x).to(device).view(B, H, S, D) for x in (Q, K, V))
    O_d = torch.zeros_like(Q_d)
    dbg_d = torch.zeros(64, dtype=torch.int32, device=device)
    flags = int(cfg["flags"])

    def launch() -> None:
        ops.fa_fwd(Q_d, K_d, V_d, causal=causal, sm_scale=sm_scale, out=O_d, flags=flags, dbg=dbg_d)

    return FabProblem(launch, O_d, dbg_d, Q, K, V, sm_scale, B, H, S, D, causal,
                      min(total_work, n_sms), (Q_d, K_d, V_d))


def fab_check(ref: Callable[..., torch.Tensor], cfg: Optional[Dict[str, object]] = None, *, B: int = 1,
              H: int = 2, S: int = 512, input_scale: float = 2.0, atol: float = 5e-2) -> bool:
    """Correctness gate on the rescale-heavy input (bench/flash_attention.jl:89-105).

    `ref(Q, K, V, sm_scale, causal)` is the per-(b,h) fp32 checker on host tensors.
    """
    p = fab_setup(B, H, S, input_scale=input_scale, cfg=cfg)
    p.launch()
    status = ops.sync_status()
    if status != 0:
        print(f"check {cfg}: device status {native.strerror(status)}")
        return False
    O = p.O_d.float().cpu().view(B * H, S, p.D)
    maxdiff = 0.0
    for i in range(B * H):
        r = slice(i * S, (i + 1) * S)
        O_ref = ref(p.Q[r], p.K[r], p.V[r], p.sm_scale, p.causal)
        maxdiff = max(maxdiff, float((O[i] - O_ref).abs().max()))
    ok = maxdiff < atol
    print(f"check {cfg}: B={B} H={H} S={S} scale={input_scale} maxdiff={maxdiff:.4g} "
          f"{'OK' if ok else 'FAIL'}")
    return ok


def fab_flops(B: int, H: int, S: int, D: int, causal: bool) -> float:
    """Forward attention work: 4*B*H*S^2*D, halved for causal (:107-108, :134)."""
    return (2.0 if causal else 4.0) * B * H * S * S * D


def fab_time(cfg: Optional[Dict[str, object]] = None, *, B: int = 1, H: int = 16, S: int = 4096,
             input_scale: float = 0.5, iters: int = 20, warmup: int = 3, warm_ms: float = 25.0):
    """Timing with the reference's warm-up discipline (:109-136), on CUDA events."""
    p = fab_setup(B, H, S, input_scale=input_scale, cfg=cfg)
    t_warm = time.perf_counter()
    launches = 0
    while launches < warmup or (time.perf_counter() - t_warm) * 1e3 < warm_ms:
        p.launch()
        launches += 1
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        p.launch()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    flops = fab_flops(B, H, S, p.D, p.causal)
    return {"ms": ms, "tflops": flops / (ms * 1e9), "ctas": p.num_ctas}


def fab_sweep(ref: Callable[..., torch.Tensor], cfgs=None,
              shapes=((1, 16, 1024), (1, 16, 2048), (1, 16, 4096), (1, 8, 8192))) -> None:
    """The standard sweep table (:140-158)."""
    cfgs = cfgs or [("default", dict(FAB_CFG_DEFAULT))]
    live = [(n, c) for n, c in cfgs if fab_check(ref, c)]
    print("shape".ljust(22) + "".join(n.ljust(22) for n, _ in live))
    for (B, H, S) in shapes:
        row = f"B={B} H={H} S={S}".ljust(22)
        for _, c in live:
            r = fab_time(c, B=B, H=H, S=S)
            row += f"{r['ms']:.3f} ms  {r['tflops']:.1f} TF".ljust(22)
        print(row)


def fab_hang_debug(cfg: Optional[Dict[str, object]] = None, *, B: int = 1, H: int = 2, S: int = 512,
                   input_scale: float = 2.0):
    """Run once and decode the device status word and CTA 0's progress counters
    (the native counterpart of the beacon decode, :163-179)."""
    p = fab_setup(B, H, S, input_scale=input_scale, cfg=cfg)
    p.launch()
    status = ops.sync_status()
    counters = p.dbg_d.cpu().tolist()[:11]
    names = ["load.kv", "mma.kv", "mma.pv0", "mma.pv1", "-", "-", "softmax0.s", "softmax1.s",
             "corr.alpha0", "corr.alpha1", "corr.items"]
    if status == 0:
        print("no timeouts -- every wait completed within the bound")
    else:
        print(native.strerror(status))
    print({n: c for n, c in zip(names, counters) if n != "-"})
    return status, counters
