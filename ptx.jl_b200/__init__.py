"""ptx.jl_b200 -- B200-native replacement for the hot path of jool-space/PTX.jl:
the tcgen05 flash-attention forward kernel and the tcgen05 bf16 GEMM under it.

The product is libptxb200.so (CUDA for sm_100a behind a C ABI, include/ptxb200.h).
This package holds its sources (csrc/), the build step, a ctypes binding, and a
host-side mirror of the reference's bench/test entry points.

The directory name contains a dot, so the package is imported under the module
name `ptx_jl_b200` through `__graft_entry__.load_package()`.
"""
from . import native  # noqa: F401  (ctypes only; does not need torch)

__all__ = ["native", "build"]


def __getattr__(name):
    # torch-dependent modules load lazily so that build/symbol checks stay light
    if name in ("ops", "flash_attention", "gemm_highperf", "rowwise", "build", "sharding"):
        import importlib
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)
