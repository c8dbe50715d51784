"""Host-side mirror of the reference's GEMM test driver.

`run_ghb(M, N, K)` follows `_run_ghb`
(test/gpu/blackwell/gemm_highperf_blackwell.jl:230-269): seeded A (M,K) and B (K,N)
~ N(0,1)*0.1, A packed K-fast, B packed as B^T (N,K) K-fast, one launch, result
returned as an (M,N) row-major tensor for the caller's checker. The native kernel
is persistent, so the reference's separate persistent driver (:491-525) maps onto
the same call.
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import ops

GHB_BM, GHB_BN, GHB_BK = 128, 256, 64   # reference tile constants (:49-51)


def ghb_inputs(M: int, N: int, K: int, *, scale: float = 0.1) -> Tuple[torch.Tensor, torch.Tensor]:
    """Host fp32 A (M,K) and B (K,N), seed formula of the reference (:232)."""
    gen = torch.Generator().manual_seed(M * 9176 + N * 131 + K)
    A = torch.randn(M, K, generator=gen) * scale
    B = torch.randn(K, N, generator=gen) * scale
    return A, B


def run_ghb(M: int, N: int, K: int, *, f32_out: bool = True, device=None):
    """Returns (D_got on host as fp32 (M,N), A, B). Raises on a device-side timeout."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    A, B = ghb_inputs(M, N, K)
    A_d = A.to(torch.bfloat16).to(device).contiguous()
    Bt_d = B.t().contiguous().to(torch.bfloat16).to(device)
    D_d = ops.gemm(A_d, Bt_d, f32_out=f32_out)
    status = ops.sync_status()
    if status != 0:
        from . import native
        raise native.PtxB200Error(status, native.strerror(status))
    return D_d.float().cpu(), A, B


def ggb_inputs(G: int, M: int, N: int, K: int, *, scale: float = 0.1) -> Tuple[torch.Tensor, torch.Tensor]:
    """Host fp32 A3 (G,M,K) and B3 (G,K,N), seed formula of the reference's grouped
    driver (test/gpu/blackwell/grouped_gemm.jl:210-212)."""
    gen = torch.Generator().manual_seed(G * 1009 + M * 997 + N * 17 + K)
    A3 = torch.randn(G, M, K, generator=gen) * scale
    B3 = torch.randn(G, K, N, generator=gen) * scale
    return A3, B3


def run_ggb(G: int, M: int, N: int, K: int, *, f32_out: bool = True, device=None):
    """Uniform grouped GEMM, the reference's `_run_ggb` (grouped_gemm.jl:208-232):
    returns (C_got on host as fp32 (G,M,N), A3, B3). Raises on a device-side timeout."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    A3, B3 = ggb_inputs(G, M, N, K)
    A_d = A3.to(torch.bfloat16).to(device).contiguous()                    # _ggb_pack_A: (G*M, K) K-fast
    Bt_d = B3.transpose(1, 2).contiguous().to(torch.bfloat16).to(device)   # _ggb_pack_B: (G*N, K) K-fast
    C_d = ops.gemm_grouped(A_d, Bt_d, f32_out=f32_out)
    status = ops.sync_status()
    if status != 0:
        from . import native
        raise native.PtxB200Error(status, native.strerror(status))
    return C_d.float().cpu(), A3, B3


def ghb_flops(M: int, N: int, K: int) -> float:
    return 2.0 * M * N * K
