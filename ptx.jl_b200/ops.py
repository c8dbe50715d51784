"""Tensor-level calls into libptxb200.so.

torch supplies device memory and streams only; each function validates what it
can on the host, then hands raw device pointers to the C ABI
(include/ptxb200.h). Nothing here computes: without the compiled library and a
compute-capability-10.x GPU these functions raise.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from . import native


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream(stream: Optional[torch.cuda.Stream], device=None) -> ctypes.c_void_p:
    s = torch.cuda.current_stream(device) if stream is None else stream
    return ctypes.c_void_p(s.cuda_stream)


def _require_cuda(*tensors) -> None:
    """Every tensor is a contiguous CUDA tensor and all of them live on one device."""
    for t in tensors:
        if not t.is_cuda:
            raise ValueError("ptxb200 ops take CUDA tensors (the library has no CPU path)")
        if not t.is_contiguous():
            raise ValueError("ptxb200 ops take contiguous tensors")
    if len({t.device for t in tensors}) > 1:
        raise ValueError("ptxb200 ops take tensors of ONE device; got " +
                         ", ".join(sorted({str(t.device) for t in tensors})))


def _check_out(out, like_device, shape, dtype, what: str = "out") -> None:
    """A caller-supplied output buffer the kernel will write `shape` elements of `dtype`
    into: anything else would be an out-of-bounds or mistyped device write."""
    _require_cuda(out)
    if out.device != like_device:
        raise ValueError(f"{what} must live on {like_device}, not {out.device}")
    if tuple(out.shape) != tuple(shape):
        raise ValueError(f"{what} must have shape {tuple(shape)}, not {tuple(out.shape)}")
    if out.dtype != dtype:
        raise ValueError(f"{what} must be {dtype}, not {out.dtype}")


def _check_stream(stream, device) -> None:
    if stream is not None and getattr(stream, "device", device) != device:
        raise ValueError(f"stream belongs to {stream.device}, the tensors to {device}")


def fa_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = False,
           sm_scale: Optional[float] = None, out: Optional[torch.Tensor] = None,
           flags: int = 0, dbg: Optional[torch.Tensor] = None,
           stream: Optional[torch.cuda.Stream] = None, lse: Optional[torch.Tensor] = None) -> torch.Tensor:
    """O = softmax(Q K^T * sm_scale [+causal]) V for [B,H,S,D] bf16 tensors
    (K, V may have fewer heads, H_kv dividing H; `lse` optionally receives the
    per-row log-sum-exp).

    Same operand layout as the reference's fab_setup (bench/flash_attention.jl:41-85):
    [B,H,S,D] row-major == a (B*H*S, D) matrix with D contiguous.
    """
    _require_cuda(q, k, v)
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise ValueError("fa_fwd takes bf16 tensors")
    if q.dim() != 4 or k.shape != v.shape or k.dim() != 4 or (q.shape[0], q.shape[2], q.shape[3]) != (
            k.shape[0], k.shape[2], k.shape[3]):
        raise ValueError("fa_fwd takes Q [B,H,S,D] and K, V [B,H_kv,S,D]")
    B, H, S, D = q.shape
    H_kv = k.shape[1]
    if lse is not None:
        _require_cuda(lse)
        if lse.device != q.device or lse.dtype != torch.float32 or lse.numel() != B * H * S:
            raise ValueError("lse must be B*H*S float32 on the tensors' device")
    if dbg is not None:
        _require_cuda(dbg)
        if dbg.device != q.device or dbg.dtype != torch.int32 or dbg.numel() < 64:
            raise ValueError("dbg must be an int32 CUDA tensor of at least 64 words on the tensors' device")
    if k.device != q.device:
        raise ValueError("q, k and v must live on one device")
    _check_stream(stream, q.device)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty_like(q)
    else:
        _check_out(out, q.device, q.shape, torch.bfloat16)
    with torch.cuda.device(q.device):
        rc = native.lib().fa_fwd_bf16_ex(_ptr(out), _ptr(lse), _ptr(q), _ptr(k), _ptr(v), B, H, H_kv, S, D,
                                         ctypes.c_float(sm_scale), int(bool(causal)), flags, _ptr(dbg),
                                         _stream(stream, q.device))
    native.check(rc)
    return out


def gemm(a: torch.Tensor, bt: torch.Tensor, *, out: Optional[torch.Tensor] = None,
         f32_out: bool = False, no_split: bool = False, one_cta: bool = False,
         stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """C[M,N] = A[M,K] @ B[K,N] with B passed column-major, i.e. as Bt = B^T [N,K].

    Operand packing of the reference's _run_ghb
    (test/gpu/blackwell/gemm_highperf_blackwell.jl:236-252).
    """
    _require_cuda(a, bt)
    if a.dtype != torch.bfloat16 or bt.dtype != torch.bfloat16:
        raise ValueError("gemm takes bf16 operands")
    if a.dim() != 2 or bt.dim() != 2 or a.shape[1] != bt.shape[1]:
        raise ValueError("gemm takes A[M,K] and Bt[N,K]")
    M, K = a.shape
    N = bt.shape[0]
    want = torch.float32 if f32_out else torch.bfloat16
    _check_stream(stream, a.device)
    if out is None:
        out = torch.empty((M, N), device=a.device, dtype=want)
        ldc = N
    else:
        # a row-strided view (columns of a wider buffer) is allowed: ldc carries the pitch
        if not out.is_cuda or out.device != a.device:
            raise ValueError(f"out must be a CUDA tensor on {a.device}")
        if out.dim() != 2 or tuple(out.shape) != (M, N) or out.stride(1) != 1 or out.stride(0) < N:
            raise ValueError(f"out must be [{M}, {N}] with unit column stride and row pitch >= {N}")
        if out.dtype != want:
            raise ValueError(f"out must be {want} (f32_out={f32_out}), not {out.dtype}")
        ldc = out.stride(0)
    flags = ((native.GEMM_F32_OUT if f32_out else 0) | (native.GEMM_NO_SPLIT if no_split else 0)
             | (native.GEMM_ONE_CTA if one_cta else 0))
    with torch.cuda.device(a.device):
        rc = native.lib().gemm_bf16(_ptr(out), _ptr(a), _ptr(bt), M, N, K, ldc, flags, _stream(stream, a.device))
    native.check(rc)
    return out


def gemm_grouped(a: torch.Tensor, bt: torch.Tensor, *, out: Optional[torch.Tensor] = None,
                 f32_out: bool = False, no_split: bool = False, one_cta: bool = False,
                 stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """C[g] = A[g] @ B[g] for A [G,M,K] and Bt [G,N,K] (each B[g] passed transposed).

    Operand packing of the reference's _run_ggb
    (test/gpu/blackwell/grouped_gemm.jl:185-232): groups stacked along the row axis.
    """
    _require_cuda(a, bt)
    if a.dtype != torch.bfloat16 or bt.dtype != torch.bfloat16:
        raise ValueError("gemm_grouped takes bf16 operands")
    if a.dim() != 3 or bt.dim() != 3 or a.shape[0] != bt.shape[0] or a.shape[2] != bt.shape[2]:
        raise ValueError("gemm_grouped takes A[G,M,K] and Bt[G,N,K]")
    G, M, K = a.shape
    N = bt.shape[1]
    want = torch.float32 if f32_out else torch.bfloat16
    _check_stream(stream, a.device)
    if out is None:
        out = torch.empty((G, M, N), device=a.device, dtype=want)
    else:
        _check_out(out, a.device, (G, M, N), want)
    flags = ((native.GEMM_F32_OUT if f32_out else 0) | (native.GEMM_NO_SPLIT if no_split else 0)
             | (native.GEMM_ONE_CTA if one_cta else 0))
    with torch.cuda.device(a.device):
        rc = native.lib().gemm_bf16_grouped(_ptr(out), _ptr(a), _ptr(bt), G, M, N, K, N, flags,
                                            _stream(stream, a.device))
    native.check(rc)
    return out


def _rowwise_check(x: torch.Tensor, *vecs: torch.Tensor) -> None:
    _require_cuda(x, *vecs)
    if x.dtype != torch.float32 or x.dim() != 2 or any(v.dtype != torch.float32 for v in vecs):
        raise ValueError("row-wise ops take a [rows, N] float32 matrix (and [N] float32 vectors)")
    if any(v.numel() != x.shape[1] for v in vecs):
        raise ValueError("weight / bias length must equal N")


def _rowwise_out(x, out, stream):
    _check_stream(stream, x.device)
    if out is None:
        return torch.empty_like(x)
    _check_out(out, x.device, x.shape, torch.float32)
    return out


def softmax(x: torch.Tensor, *, out: Optional[torch.Tensor] = None,
            stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """Row-wise softmax of a [rows, N] float32 matrix (test/gpu/softmax.jl:151-163)."""
    _rowwise_check(x)
    out = _rowwise_out(x, out, stream)
    with torch.cuda.device(x.device):
        rc = native.lib().softmax_f32(_ptr(out), _ptr(x), x.shape[0], x.shape[1], _stream(stream, x.device))
    native.check(rc)
    return out


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6, *, out: Optional[torch.Tensor] = None,
             stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """y = x * w / sqrt(mean(x^2) + eps) per row (test/gpu/rms_norm.jl:121-139)."""
    _rowwise_check(x, w)
    out = _rowwise_out(x, out, stream)
    with torch.cuda.device(x.device):
        rc = native.lib().rms_norm_f32(_ptr(out), _ptr(x), _ptr(w), x.shape[0], x.shape[1],
                                       ctypes.c_float(eps), _stream(stream, x.device))
    native.check(rc)
    return out


def layer_norm(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor, eps: float = 1e-5, *,
               out: Optional[torch.Tensor] = None,
               stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """y = (x - mean) / sqrt(var + eps) * w + bias per row (test/gpu/layer_norm.jl:138-156)."""
    _rowwise_check(x, w, bias)
    out = _rowwise_out(x, out, stream)
    with torch.cuda.device(x.device):
        rc = native.lib().layer_norm_f32(_ptr(out), _ptr(x), _ptr(w), _ptr(bias), x.shape[0],
                                         x.shape[1], ctypes.c_float(eps), _stream(stream, x.device))
    native.check(rc)
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor, *, out: Optional[torch.Tensor] = None,
           stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """out = silu(gate) * up elementwise, float32 (test/gpu/swiglu.jl:77-98)."""
    _require_cuda(gate, up)
    if gate.dtype != torch.float32 or up.dtype != torch.float32 or gate.shape != up.shape:
        raise ValueError("swiglu takes two float32 tensors of one shape")
    out = _rowwise_out(gate, out, stream)
    with torch.cuda.device(gate.device):
        rc = native.lib().swiglu_f32(_ptr(out), _ptr(gate), _ptr(up), gate.numel(), _stream(stream, gate.device))
    native.check(rc)
    return out


def selftest(which: int, q=None, k=None, v=None, p=None):
    """Run bring-up probe `which` (see ptxb200_selftest). Returns (out_s, out_o)."""
    dev = torch.device("cuda", torch.cuda.current_device())
    if which == 0:
        out_s = torch.zeros(128 * 128, dtype=torch.int32, device=dev)
        rc = native.lib().ptxb200_selftest(0, _ptr(out_s), None, None, None, None, None, _stream(None))
        native.check(rc)
        return out_s.view(128, 128), None
    if which == 3 or which == 4:
        out_s = torch.zeros(16, dtype=torch.int32, device=dev)
        rc = native.lib().ptxb200_selftest(which, _ptr(out_s), None, None, None, None, None, _stream(None))
        native.check(rc)
        return out_s, None
    D = 128 if which == 1 else 64
    _require_cuda(q, k, v, p)
    out_s = torch.zeros((128, 128), dtype=torch.float32, device=dev)
    out_o = torch.zeros((128, D), dtype=torch.float32, device=dev)
    rc = native.lib().ptxb200_selftest(which, _ptr(out_s), _ptr(out_o), _ptr(q), _ptr(k), _ptr(v),
                                       _ptr(p), _stream(None))
    native.check(rc)
    return out_s, out_o


def sync_status(stream: Optional[torch.cuda.Stream] = None) -> int:
    """0 = healthy. With a stream: synchronise it and return (and clear) its status word.
    Without: synchronise the current device and return (and clear) the first nonzero
    status of ANY stream that launched through the library on it."""
    if stream is None:
        return native.device_status()
    with torch.cuda.device(stream.device):
        return native.sync_status(stream.cuda_stream)
