"""Helpers shared by the parity tests."""
import numpy as np
import torch

# Acceptance tolerance of the hot path against the fp32 oracle
# (tighter than the reference's own gate of max abs < 5e-2,
# test/gpu/blackwell/flash_attention.jl:207,220).
ATTN_MAX_ABS = 2e-2
ATTN_MEAN_ABS = 2e-3


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16 tensor (any device) -> uint16 numpy array of the same shape."""
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def seeded_qkv(B, H, S, D, seed, sigma_qk=1.0, sigma_v=1.0):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, H, S, D, generator=g) * sigma_qk).to(torch.bfloat16)
    k = (torch.randn(B, H, S, D, generator=g) * sigma_qk).to(torch.bfloat16)
    v = (torch.randn(B, H, S, D, generator=g) * sigma_v).to(torch.bfloat16)
    return q, k, v


def attn_errors(o_dev: torch.Tensor, ref: np.ndarray):
    got = o_dev.float().cpu().numpy().reshape(ref.shape)
    err = np.abs(got - ref)
    return float(err.max()), float(err.mean())
