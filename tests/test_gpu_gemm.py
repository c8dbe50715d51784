"""gemm_bf16 parity against the CPU oracle, through the C ABI.

Shapes and tolerance of the reference's own runtime tests
(test/gpu/blackwell/gemm_highperf_blackwell.jl:271-277, 533-539:
isapprox(rtol=5e-2, atol=5e-2)); here the bound is far tighter because both sides
accumulate bf16 products in fp32.
"""
import numpy as np
import pytest
import torch

from util import bits

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [
    (128, 256, 64),      # 1 tile, 1 K-iteration (< ring depth)
    (128, 256, 512),     # 1 tile, 8 K-iterations (ring slot reuse)
    (256, 512, 256),     # 2x2 tiles
    (128, 128, 64),      # N smaller than the 256-wide tile (zero-filled box, guarded stores)
    (384, 640, 192),     # ragged: N % 256 == 128, odd tile counts
    (2048, 4096, 1024),  # more tiles than SMs: several tiles per persistent CTA
])
@pytest.mark.parametrize("f32_out", [True, False])
def test_gemm_matches_oracle(pkg, gpu, oracle_mod, M, N, K, f32_out):
    gm = pkg.gemm_highperf
    A, B = gm.ghb_inputs(M, N, K)
    a = A.to(torch.bfloat16)
    bt = B.t().contiguous().to(torch.bfloat16)
    c = pkg.ops.gemm(a.to(gpu), bt.to(gpu), f32_out=f32_out)
    assert pkg.ops.sync_status() == 0
    ref = oracle_mod.gemm_ref_c(bits(a), bits(bt))
    got = c.float().cpu().numpy()
    if f32_out:
        np.testing.assert_allclose(got, ref, rtol=1e-4, atol=1e-4)
    else:
        # one bf16 rounding of the fp32 result: relative 2^-8
        np.testing.assert_allclose(got, ref, rtol=2 ** -7, atol=1e-3)


def test_gemm_ldc_and_linearity(pkg, gpu):
    """Size-independent properties at a large shape: C written with ldc > N leaves
    the padding untouched, and A*(B1+B2) == A*B1 + A*B2 up to rounding."""
    M, N, K = 1024, 1024, 2048
    g = torch.Generator().manual_seed(5)
    a = (torch.randn(M, K, generator=g) * 0.1).to(torch.bfloat16).to(gpu)
    b1 = (torch.randint(-4, 5, (N, K), generator=g).float() / 8).to(torch.bfloat16).to(gpu)
    b2 = (torch.randint(-4, 5, (N, K), generator=g).float() / 8).to(torch.bfloat16).to(gpu)
    buf = torch.full((M, N + 64), 7.0, dtype=torch.float32, device=gpu)
    out = buf[:, :N]
    rc = pkg.native.lib().gemm_bf16(out.data_ptr(), a.data_ptr(), b1.data_ptr(), M, N, K, N + 64,
                                    pkg.native.GEMM_F32_OUT, torch.cuda.current_stream().cuda_stream)
    assert rc == 0 and pkg.ops.sync_status() == 0
    assert torch.all(buf[:, N:] == 7.0)
    c1 = buf[:, :N].clone()
    c2 = pkg.ops.gemm(a, b2, f32_out=True)
    c12 = pkg.ops.gemm(a, (b1 + b2), f32_out=True)   # b1+b2 is exact in bf16 (small dyadic values)
    assert pkg.ops.sync_status() == 0
    torch.testing.assert_close(c12, c1 + c2, rtol=1e-4, atol=1e-3)


def test_gemm_rejects_bad_arguments(pkg, gpu):
    L = pkg.native.lib()
    a = torch.zeros(128, 64, dtype=torch.bfloat16, device=gpu)
    c = torch.zeros(128, 128, dtype=torch.bfloat16, device=gpu)
    P = lambda t: t.data_ptr()
    assert L.gemm_bf16(P(c), P(a), P(a), 100, 128, 64, 128, 0, None) == pkg.native.E_SHAPE
    assert L.gemm_bf16(P(c), P(a), P(a), 128, 128, 32, 128, 0, None) == pkg.native.E_SHAPE
    assert L.gemm_bf16(None, P(a), P(a), 128, 128, 64, 128, 0, None) == pkg.native.E_INVALID
    assert L.gemm_bf16(P(c), P(a) + 2, P(a), 128, 128, 64, 128, 0, None) == pkg.native.E_ALIGN
    assert L.gemm_bf16(P(c), P(a), P(a), 128, 128, 64, 64, 0, None) == pkg.native.E_INVALID
