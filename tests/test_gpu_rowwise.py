"""Row-wise fp32 kernels (softmax, RMS norm, layer norm, SwiGLU) against the float64
restatements of the reference's CPU references, through the C ABI.

Shapes, seeds, input distributions and the tolerance (atol 1e-4, rtol 1e-3) are the
reference's own (test/gpu/softmax.jl:151-163, rms_norm.jl:121-139,
layer_norm.jl:138-156, swiglu.jl:77-98); further shapes cover each threads-per-row
regime of the native kernels, ragged rows (N % 128 != 0), one row, and sizes far
beyond L2 through properties that need no oracle.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ATOL, RTOL = 1e-4, 1e-3

# (rows, N): reference shapes, then 1 / 2 / 16 accesses per lane with one warp per row,
# ragged widths, the 256- and 1024-thread regimes and their edges, the largest N.
SHAPES = [(4, 512), (8, 1024), (16, 2048), (3, 4), (5, 132), (7, 260), (1, 2048), (9, 2052),
          (33, 4096), (6, 8192), (5, 8196), (4, 20000), (3, 32768), (1000, 768), (5000, 1536)]


@pytest.mark.parametrize("B,N", SHAPES)
def test_softmax_matches_oracle(pkg, gpu, oracle_mod, B, N):
    Y, X = pkg.rowwise.run_softmax(B, N, device=gpu)
    ref = oracle_mod.softmax_ref_numpy(X.numpy())
    np.testing.assert_allclose(Y.numpy(), ref, atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("B,N", SHAPES)
def test_rms_norm_matches_oracle(pkg, gpu, oracle_mod, B, N):
    Y, X, W = pkg.rowwise.run_rms_norm(B, N, device=gpu)
    ref = oracle_mod.rms_norm_ref_numpy(X.numpy(), W.numpy(), 1e-6)
    np.testing.assert_allclose(Y.numpy(), ref, atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("B,N", SHAPES)
def test_layer_norm_matches_oracle(pkg, gpu, oracle_mod, B, N):
    Y, X, W, Bias = pkg.rowwise.run_layer_norm(B, N, device=gpu)
    ref = oracle_mod.layer_norm_ref_numpy(X.numpy(), W.numpy(), Bias.numpy(), 1e-5)
    np.testing.assert_allclose(Y.numpy(), ref, atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("M,F", [(4, 512), (32, 1024), (8, 2048), (1, 4), (3, 36), (257, 1028), (4096, 5504)])
def test_swiglu_matches_oracle(pkg, gpu, oracle_mod, M, F):
    out, gate, up = pkg.rowwise.run_swiglu(M, F, device=gpu)
    ref = oracle_mod.swiglu_ref_numpy(gate.numpy(), up.numpy())
    assert np.max(np.abs(out.numpy() - ref)) < 1e-4          # swiglu.jl:95-96
    np.testing.assert_allclose(out.numpy(), ref, atol=ATOL, rtol=RTOL)


def test_layer_norm_large_mean(pkg, gpu, oracle_mod):
    """Rows whose mean dwarfs their spread: the variance comes from centred values,
    so the result keeps its accuracy where E[x^2] - mean^2 would cancel."""
    g = torch.Generator().manual_seed(3)
    X = torch.randn(64, 4096, generator=g) * 0.05 + 300.0
    W = torch.ones(4096)
    Bias = torch.zeros(4096)
    Y = pkg.ops.layer_norm(X.to(gpu), W.to(gpu), Bias.to(gpu), 1e-5).cpu()
    assert pkg.ops.sync_status() == 0
    ref = oracle_mod.layer_norm_ref_numpy(X.numpy(), W.numpy(), Bias.numpy(), 1e-5)
    np.testing.assert_allclose(Y.numpy(), ref, atol=5e-3, rtol=5e-3)   # fp32 input spacing at 300 is 3e-5 of a 0.05 spread


def test_rowwise_properties_at_full_size(pkg, gpu):
    """1 GiB in, 1 GiB out per call: softmax rows sum to one and do not move under a
    row shift; RMS norm is invariant to a positive row scale; layer norm output has
    zero mean and unit variance; SwiGLU is odd-symmetric in the way silu allows."""
    rows, N = 65536, 4096
    g = torch.Generator(device=gpu).manual_seed(7)
    X = torch.randn(rows, N, generator=g, device=gpu)
    Y = pkg.ops.softmax(X)
    assert torch.allclose(Y.sum(dim=1), torch.ones(rows, device=gpu), atol=1e-4)
    assert float(Y.min()) >= 0.0
    shift = torch.randn(rows, 1, generator=g, device=gpu) * 4
    Y2 = pkg.ops.softmax(X + shift)
    torch.testing.assert_close(Y2, Y, atol=1e-6, rtol=2e-3)
    del Y2
    W = torch.rand(N, generator=g, device=gpu) + 0.5
    R1 = pkg.ops.rms_norm(X, W, 0.0)
    R2 = pkg.ops.rms_norm(X * 8.0, W, 0.0)     # exact scaling by a power of two
    torch.testing.assert_close(R2, R1, atol=1e-6, rtol=1e-5)
    del R1, R2
    L = pkg.ops.layer_norm(X, torch.ones(N, device=gpu), torch.zeros(N, device=gpu), 0.0)
    assert float(L.mean(dim=1).abs().max()) < 1e-5
    assert float((L.var(dim=1, unbiased=False) - 1.0).abs().max()) < 1e-4
    del L
    U = torch.randn(rows, N, generator=g, device=gpu)
    S1 = pkg.ops.swiglu(X, U)
    S2 = pkg.ops.swiglu(-X, U)
    # silu(x) - silu(-x) = x, so swiglu(x,u) - swiglu(-x,u) = x*u
    torch.testing.assert_close(S1 - S2, X * U, atol=2e-5, rtol=2e-3)
    assert pkg.ops.sync_status() == 0


def test_rowwise_bad_arguments(pkg, gpu):
    n = pkg.native
    L = n.lib()
    x = torch.zeros(8, 64, device=gpu)
    p = x.data_ptr()
    st = torch.cuda.current_stream().cuda_stream
    import ctypes
    eps = ctypes.c_float(1e-6)
    assert L.softmax_f32(p, p, 8, 66, st) == n.E_SHAPE          # N % 4
    assert L.softmax_f32(p, p, 8, 32772, st) == n.E_SHAPE       # beyond the register-resident row
    assert L.softmax_f32(p, p, 0, 64, st) == n.E_INVALID
    assert L.softmax_f32(p, p + 4, 8, 64, st) == n.E_ALIGN
    assert L.rms_norm_f32(p, p, None, 8, 64, eps, st) == n.E_INVALID
    assert L.layer_norm_f32(p, p, p, None, 8, 64, eps, st) == n.E_INVALID
    assert L.rms_norm_f32(p, p, p, 8, 64, ctypes.c_float(-1.0), st) == n.E_INVALID
    assert L.swiglu_f32(p, p, p, 6, st) == n.E_SHAPE
    assert L.swiglu_f32(p, p, None, 8, st) == n.E_INVALID
