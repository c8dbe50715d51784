"""ctypes binding of libptxb200.so (the C ABI declared in include/ptxb200.h).

There is no fallback: if the shared library is missing or does not load, every
call raises. Device memory, streams and multi-process plumbing come from
PyTorch; the arithmetic happens only inside the library's CUDA kernels.
"""
from __future__ import annotations

import ctypes
import os
import re
from typing import List, Optional

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
# PTXB200_LIB_PATH overrides the in-tree library (e.g. an instrumented build)
LIB_PATH = os.environ.get("PTXB200_LIB_PATH") or os.path.join(PKG_DIR, "libptxb200.so")
HEADER_PATH = os.path.join(PKG_DIR, "..", "include", "ptxb200.h")

GEMM_F32_OUT = 0x1
GEMM_NO_SPLIT = 0x2
GEMM_ONE_CTA = 0x4
FA_NO_LAZY_RESCALE = 0x1
FA_SINGLE_BLOCKS = 0x2
FA_NO_TAIL_SPLIT = 0x4
FA_ALWAYS_TAIL_SPLIT = 0x8

E_INVALID, E_SHAPE, E_ALIGN, E_CUDA, E_DRIVER, E_DEVICE, E_CAPACITY = -1, -2, -3, -4, -5, -6, -7


class PtxB200Error(RuntimeError):
    """A nonzero return code from the library."""

    def __init__(self, code: int, text: str):
        super().__init__(f"ptxb200 error {code}: {text}")
        self.code = code


_lib: Optional[ctypes.CDLL] = None


def declared_symbols() -> List[str]:
    """Names of every function include/ptxb200.h declares."""
    with open(HEADER_PATH) as f:
        text = f.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"^\s*(?:const\s+char\s*\*|int)\s+(\w+)\s*\(", text, flags=re.M)


def lib() -> ctypes.CDLL:
    """Load the shared library (once) and set the argument types."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise PtxB200Error(-100, f"{LIB_PATH} is missing; run `python -m __graft_entry__` "
                                 "or ptx.jl_b200/build.py to compile it (there is no fallback path)")
    L = ctypes.CDLL(LIB_PATH)
    vp, ci, cu, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_float
    L.ptxb200_version.restype = ci
    L.ptxb200_version.argtypes = []
    L.ptxb200_strerror.restype = ctypes.c_char_p
    L.ptxb200_strerror.argtypes = [ci]
    L.ptxb200_last_cuda_error.restype = ctypes.c_char_p
    L.ptxb200_last_cuda_error.argtypes = []
    L.gemm_bf16.restype = ci
    L.gemm_bf16.argtypes = [vp, vp, vp, ci, ci, ci, ci, cu, vp]
    L.softmax_f32.restype = ci
    L.softmax_f32.argtypes = [vp, vp, ci, ci, vp]
    L.rms_norm_f32.restype = ci
    L.rms_norm_f32.argtypes = [vp, vp, vp, ci, ci, ctypes.c_float, vp]
    L.layer_norm_f32.restype = ci
    L.layer_norm_f32.argtypes = [vp, vp, vp, vp, ci, ci, ctypes.c_float, vp]
    L.swiglu_f32.restype = ci
    L.swiglu_f32.argtypes = [vp, vp, vp, ctypes.c_longlong, vp]
    L.gemm_bf16_grouped.restype = ci
    L.gemm_bf16_grouped.argtypes = [vp, vp, vp, ci, ci, ci, ci, ci, cu, vp]
    L.fa_fwd_bf16.restype = ci
    L.fa_fwd_bf16.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, cf, ci, cu, vp, vp]
    L.fa_fwd_bf16_ex.restype = ci
    L.fa_fwd_bf16_ex.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, cf, ci, cu, vp, vp]
    L.fa_fwd_bf16_noalloc.restype = ci
    L.fa_fwd_bf16_noalloc.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, cf, ci, cu, vp]
    L.fa_fwd_bf16_noalloc_status.restype = ci
    L.fa_fwd_bf16_noalloc_status.argtypes = [vp, ci, vp]
    L.ptxb200_sync_status.restype = ci
    L.ptxb200_sync_status.argtypes = [vp]
    L.ptxb200_fa_plan.restype = ci
    L.ptxb200_fa_plan.argtypes = [ci, ci, ci, ci, cu, ci, vp, ci]
    L.ptxb200_device_status.restype = ci
    L.ptxb200_device_status.argtypes = []
    L.ptxb200_selftest.restype = ci
    L.ptxb200_selftest.argtypes = [ci, vp, vp, vp, vp, vp, vp, vp]
    L.ptxb200_shutdown.restype = ci
    L.ptxb200_shutdown.argtypes = []
    _lib = L
    return L


def strerror(code: int) -> str:
    text = lib().ptxb200_strerror(code).decode()
    if code == E_CUDA or code == E_DRIVER:
        text += " -- " + lib().ptxb200_last_cuda_error().decode()
    return text


def check(code: int) -> None:
    if code != 0:
        raise PtxB200Error(code, strerror(code))


def sync_status(stream: int = 0) -> int:
    """Synchronise the stream and return (and clear) its status word."""
    return lib().ptxb200_sync_status(ctypes.c_void_p(stream))


def device_status() -> int:
    """Synchronise the current device and return (and clear) the first nonzero status
    word of any stream that launched through the library on it."""
    return lib().ptxb200_device_status()
