"""Host-side mirror of the reference's row-wise kernel test drivers.

Each `run_*` follows the corresponding testset body
(test/gpu/softmax.jl:151-163, test/gpu/rms_norm.jl:121-139,
test/gpu/layer_norm.jl:138-156, test/gpu/swiglu.jl:77-98): seeded inputs of the same
distributions and seed formulas, the matrix flattened row-major, one launch, the
result returned on the host for the caller's checker. The reference's `block`
argument (threads per row, a compile-time value there) has no counterpart: the
native kernels pick the threads per row from N.
"""
from __future__ import annotations

import torch

from . import native, ops

REFERENCE_SHAPES = [(4, 512), (8, 1024), (16, 2048)]          # (rows, N) of the norm/softmax testsets
REFERENCE_SWIGLU_SHAPES = [(4, 512), (32, 1024), (8, 2048)]   # (M, F)


def _checked(t: torch.Tensor) -> torch.Tensor:
    status = ops.sync_status()
    if status != 0:
        raise native.PtxB200Error(status, native.strerror(status))
    return t.cpu()


def softmax_inputs(B: int, N: int) -> torch.Tensor:
    gen = torch.Generator().manual_seed(B * 7919 + N)          # softmax.jl:154
    return torch.randn(B, N, generator=gen)


def run_softmax(B: int, N: int, device=None):
    device = device or torch.device("cuda", torch.cuda.current_device())
    X = softmax_inputs(B, N)
    return _checked(ops.softmax(X.to(device))), X


def rms_norm_inputs(B: int, N: int):
    gen = torch.Generator().manual_seed(B * 7919 + N)          # rms_norm.jl:125-127
    X = torch.randn(B, N, generator=gen) * 0.3
    W = torch.randn(N, generator=gen) * 0.1 + 1.0
    return X, W


def run_rms_norm(B: int, N: int, eps: float = 1e-6, device=None):
    device = device or torch.device("cuda", torch.cuda.current_device())
    X, W = rms_norm_inputs(B, N)
    return _checked(ops.rms_norm(X.to(device), W.to(device), eps)), X, W


def layer_norm_inputs(B: int, N: int):
    gen = torch.Generator().manual_seed(B * 65537 + N)         # layer_norm.jl:142-145
    X = torch.randn(B, N, generator=gen) * 2.0 - 1.0
    W = torch.randn(N, generator=gen) * 0.1 + 1.0
    Bias = torch.randn(N, generator=gen) * 0.1
    return X, W, Bias


def run_layer_norm(B: int, N: int, eps: float = 1e-5, device=None):
    device = device or torch.device("cuda", torch.cuda.current_device())
    X, W, Bias = layer_norm_inputs(B, N)
    return _checked(ops.layer_norm(X.to(device), W.to(device), Bias.to(device), eps)), X, W, Bias


def swiglu_inputs(M: int, F: int):
    gen = torch.Generator().manual_seed(M * 65537 + F)         # swiglu.jl:80-82
    gate = torch.randn(M * F, generator=gen) * 0.5
    up = torch.randn(M * F, generator=gen) * 0.5
    return gate, up


def run_swiglu(M: int, F: int, device=None):
    device = device or torch.device("cuda", torch.cuda.current_device())
    gate, up = swiglu_inputs(M, F)
    return _checked(ops.swiglu(gate.to(device), up.to(device))), gate, up
