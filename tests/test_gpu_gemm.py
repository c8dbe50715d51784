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


# ---------------------------------------------------------------------------
# gemm_bf16_grouped: the reference's uniform grouped GEMM
# (test/gpu/blackwell/grouped_gemm.jl:234-244: (G,M,N,K) = (1,128,64,64),
# (2,128,64,64), (4,128,64,128), isapprox(rtol=5e-2, atol=5e-2) against a bf16
# CPU reference), plus shapes whose column tiles straddle groups or fill several
# persistent rounds.
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("G,M,N,K", [
    (1, 128, 64, 64),
    (2, 128, 64, 64),
    (4, 128, 64, 128),
    (3, 256, 192, 192),    # N % 256 != 0: every B^T box reaches into the next group
    (5, 128, 320, 64),     # two column tiles per group, the second one ragged
    (8, 512, 1024, 512),   # 8 * 4 * 4 = 128 tiles
    (16, 1024, 512, 256),  # 256 tiles: more than one round per CTA
])
@pytest.mark.parametrize("f32_out", [True, False])
def test_grouped_gemm_matches_oracle(pkg, gpu, oracle_mod, G, M, N, K, f32_out):
    gm = pkg.gemm_highperf
    A3, B3 = gm.ggb_inputs(G, M, N, K)
    a = A3.to(torch.bfloat16)
    bt = B3.transpose(1, 2).contiguous().to(torch.bfloat16)
    c = pkg.ops.gemm_grouped(a.to(gpu), bt.to(gpu), f32_out=f32_out)
    assert pkg.ops.sync_status() == 0
    got = c.float().cpu().numpy()
    for g in range(G):
        ref = oracle_mod.gemm_ref_c(bits(a[g]), bits(bt[g]))
        if f32_out:
            np.testing.assert_allclose(got[g], ref, rtol=1e-4, atol=1e-4)
        else:
            np.testing.assert_allclose(got[g], ref, rtol=2 ** -7, atol=1e-3)


def test_grouped_gemm_equals_per_group_calls(pkg, gpu):
    """The grouped launch runs the same arithmetic per tile as one gemm_bf16 call per
    group: results are bit-identical, a poisoned neighbour group leaks nowhere, and
    padding behind ldc stays untouched."""
    G, M, N, K = 6, 256, 192, 320
    g = torch.Generator().manual_seed(11)
    a = (torch.randn(G, M, K, generator=g) * 0.1).to(torch.bfloat16).to(gpu)
    bt = (torch.randn(G, N, K, generator=g) * 0.1).to(torch.bfloat16).to(gpu)
    bt[3] = float("nan")   # group 3's B: only group 3's C may see it
    buf = torch.full((G * M, N + 32), 7.0, dtype=torch.float32, device=gpu)
    # NO_SPLIT: with tiles cut along K the summation order depends on the tile count
    rc = pkg.native.lib().gemm_bf16_grouped(buf.data_ptr(), a.data_ptr(), bt.data_ptr(), G, M, N, K,
                                            N + 32, pkg.native.GEMM_F32_OUT | pkg.native.GEMM_NO_SPLIT,
                                            torch.cuda.current_stream().cuda_stream)
    assert rc == 0 and pkg.ops.sync_status() == 0
    assert torch.all(buf[:, N:] == 7.0)
    got = buf[:, :N].reshape(G, M, N)
    for i in range(G):
        if i == 3:
            assert torch.isnan(got[i]).all()
            continue
        # N = 192 is outside gemm_bf16's N % 128 contract: compare on a 128-column slice
        one = pkg.ops.gemm(a[i], bt[i, :128].contiguous(), f32_out=True, no_split=True)
        assert torch.equal(got[i][:, :128], one)
        assert torch.isfinite(got[i]).all()
    assert pkg.ops.sync_status() == 0


# ---------------------------------------------------------------------------
# Tiles cut along K (no reference counterpart): at most half as many tiles as SMs,
# K long enough for the split to pay.
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K", [
    (128, 256, 8192),     # one tile shared by 16 CTAs
    (128, 128, 4096),     # one ragged tile
    (256, 512, 4096),     # 4 tiles, 32 CTAs, 8 iterations each
    (384, 768, 2048),     # 9 tiles: shares cross tile boundaries unevenly
    (1024, 1024, 8192),   # 32 tiles on 148 CTAs: most CTAs hold two partial tiles
    (1152, 2048, 4096),   # 72 tiles, just under half the SMs
    (2048, 4096, 8192),   # 256 tiles: not split (the flag then changes nothing)
])
@pytest.mark.parametrize("f32_out", [True, False])
def test_gemm_split_tail_matches_oracle_and_unsplit(pkg, gpu, oracle_mod, M, N, K, f32_out):
    g = torch.Generator().manual_seed(M + N + K)
    a = (torch.randn(M, K, generator=g) * 0.1).to(torch.bfloat16)
    bt = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16)
    a_d, bt_d = a.to(gpu), bt.to(gpu)
    c = pkg.ops.gemm(a_d, bt_d, f32_out=f32_out)
    c_again = pkg.ops.gemm(a_d, bt_d, f32_out=f32_out)
    c_whole = pkg.ops.gemm(a_d, bt_d, f32_out=f32_out, no_split=True)
    assert pkg.ops.sync_status() == 0
    assert torch.equal(c, c_again)                       # fixed summation order: reproducible
    # against the unsplit order: fp32 re-association only
    torch.testing.assert_close(c.float(), c_whole.float(), rtol=2 ** -7 if not f32_out else 1e-4, atol=1e-3)
    if M * N * K <= 2 ** 33:
        ref = oracle_mod.gemm_ref_c(bits(a), bits(bt))
        got = c.float().cpu().numpy()
        if f32_out:
            np.testing.assert_allclose(got, ref, rtol=1e-4, atol=1e-4)
        else:
            np.testing.assert_allclose(got, ref, rtol=2 ** -7, atol=1e-3)


def test_grouped_gemm_split_tail(pkg, gpu):
    """Groups and the K split compose: 10 groups x 3 tiles shared by 148 CTAs."""
    G, M, N, K = 10, 128, 768, 4096
    g = torch.Generator().manual_seed(77)
    a = (torch.randn(G, M, K, generator=g) * 0.1).to(torch.bfloat16).to(gpu)
    bt = (torch.randn(G, N, K, generator=g) * 0.1).to(torch.bfloat16).to(gpu)
    c = pkg.ops.gemm_grouped(a, bt, f32_out=True)
    ref = torch.bmm(a.float(), bt.float().transpose(1, 2))
    assert pkg.ops.sync_status() == 0
    torch.testing.assert_close(c, ref, rtol=1e-4, atol=1e-3)


def test_gemm_split_on_two_streams(pkg, gpu):
    """Scratch is per stream: split launches that overlap on two streams stay correct."""
    M, N, K = 256, 512, 8192
    g = torch.Generator().manual_seed(9)
    a = (torch.randn(M, K, generator=g) * 0.1).to(torch.bfloat16).to(gpu)
    bts = [(torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16).to(gpu) for _ in range(2)]
    want = [pkg.ops.gemm(a, bt, f32_out=True) for bt in bts]
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    outs = [torch.empty(M, N, device=gpu) for _ in range(2)]
    for _ in range(20):
        for st, bt, o in zip(streams, bts, outs):
            pkg.ops.gemm(a, bt, out=o, f32_out=True, stream=st)
    torch.cuda.synchronize()
    assert pkg.ops.sync_status() == 0
    for o, w in zip(outs, want):
        assert torch.equal(o, w)


# ---------------------------------------------------------------------------
# CTA-pair kernel (256x256 tile per pair of SMs, tcgen05.mma.cta_group::2): taken when
# there are at least 74 such tiles (the last row-tile may be half-filled). Same k-order per output element
# as the one-CTA kernel, so the two must agree bit for bit.
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K", [
    (2048, 4096, 1024),   # 8 x 16 tiles: two rounds for most pairs
    (4096, 2176, 256),    # N % 256 == 128: zero-filled half boxes, guarded stores
    (2560, 2048, 64),     # a single k-iteration per tile (ring shorter than its depth)
    (2432, 2304, 128),    # M % 256 == 128: the last row-tile is half-filled (peer rows not stored)
    (8192, 8192, 512),    # 1024 tiles
])
@pytest.mark.parametrize("f32_out", [True, False])
def test_gemm_pair_kernel_equals_one_cta_kernel(pkg, gpu, oracle_mod, M, N, K, f32_out):
    g = torch.Generator().manual_seed(M * 3 + N * 5 + K)
    a = (torch.randn(M, K, generator=g) * 0.1).to(torch.bfloat16)
    bt = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16)
    a_d, bt_d = a.to(gpu), bt.to(gpu)
    c_pair = pkg.ops.gemm(a_d, bt_d, f32_out=f32_out)
    c_one = pkg.ops.gemm(a_d, bt_d, f32_out=f32_out, one_cta=True)
    assert pkg.ops.sync_status() == 0
    assert torch.equal(c_pair, c_one)
    if M * N * K <= 2 ** 33:
        ref = oracle_mod.gemm_ref_c(bits(a), bits(bt))
        got = c_pair.float().cpu().numpy()
        if f32_out:
            np.testing.assert_allclose(got, ref, rtol=1e-4, atol=1e-4)
        else:
            np.testing.assert_allclose(got, ref, rtol=2 ** -7, atol=1e-3)


def test_grouped_gemm_pair_kernel(pkg, gpu):
    G, M, N, K = 4, 1152, 1280, 256     # 4 x 5 x 5 = 100 tiles of 256 x 256, each group's last row-tile half-filled
    g = torch.Generator().manual_seed(21)
    a = (torch.randn(G, M, K, generator=g) * 0.1).to(torch.bfloat16).to(gpu)
    bt = (torch.randn(G, N, K, generator=g) * 0.1).to(torch.bfloat16).to(gpu)
    c_pair = pkg.ops.gemm_grouped(a, bt, f32_out=True)
    c_one = pkg.ops.gemm_grouped(a, bt, f32_out=True, one_cta=True)
    assert pkg.ops.sync_status() == 0
    assert torch.equal(c_pair, c_one)
    torch.testing.assert_close(c_pair, torch.bmm(a.float(), bt.float().transpose(1, 2)), rtol=1e-4, atol=1e-3)


def _random_gemm_shapes(n, seed):
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(n):
        M = 128 * int(rng.integers(1, 25))
        N = 128 * int(rng.integers(1, 25))
        K = 64 * int(rng.integers(1, 49))
        out.append((M, N, K))
    return out


@pytest.mark.parametrize("M,N,K", _random_gemm_shapes(12, 20260026))
def test_gemm_seeded_random_shapes(pkg, gpu, oracle_mod, M, N, K):
    """Shapes drawn from a seeded generator, so that whichever schedule the dispatch picks
    (one-CTA persistent, split along K, CTA pair) is checked against the oracle, and
    against the one-CTA kernel without a split: bit for bit where the k-order per element
    is the same (no split), to fp32 summation-order tolerance where it is not."""
    g = torch.Generator().manual_seed(M * 7 + N * 3 + K)
    a = (torch.randn(M, K, generator=g) * 0.1).to(torch.bfloat16)
    bt = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16)
    a_d, bt_d = a.to(gpu), bt.to(gpu)
    c = pkg.ops.gemm(a_d, bt_d, f32_out=True)
    c_plain = pkg.ops.gemm(a_d, bt_d, f32_out=True, no_split=True, one_cta=True)
    c_nosplit = pkg.ops.gemm(a_d, bt_d, f32_out=True, no_split=True)
    status = pkg.ops.sync_status()
    assert status == 0, pkg.native.strerror(status)
    assert torch.equal(c_nosplit, c_plain)
    torch.testing.assert_close(c, c_plain, rtol=1e-4, atol=1e-4)
    ref = oracle_mod.gemm_ref_c(bits(a), bits(bt))
    np.testing.assert_allclose(c.cpu().numpy(), ref, rtol=1e-4, atol=1e-4)


# ---------------------------------------------------------------------------
# The full-size GEMM configuration: M = N = K = 8192, entries uniform in [-1, 1], bf16
# out. The oracle cannot form all of C in test time, so 256 x 256 blocks of C are checked
# against it over the full K: the four corners, the centre, and blocks drawn from a
# seeded generator (the reference checks the whole of its small C the same way:
# test/gpu/blackwell/gemm_highperf_blackwell.jl:224-228, 257-262).
# ---------------------------------------------------------------------------
def _c5_blocks(n_random, seed, tiles=8192 // 256):
    rng = np.random.default_rng(seed)
    blocks = [(0, 0), (0, tiles - 1), (tiles - 1, 0), (tiles - 1, tiles - 1), (tiles // 2, tiles // 2)]
    while len(blocks) < 5 + n_random:
        b = (int(rng.integers(0, tiles)), int(rng.integers(0, tiles)))
        if b not in blocks:
            blocks.append(b)
    return blocks


@pytest.mark.parametrize("one_cta", [False, True], ids=["cta_pair", "one_cta"])
def test_gemm_full_size_uniform_inputs_bf16_out(pkg, gpu, oracle_mod, one_cta):
    M = N = K = 8192
    g = torch.Generator().manual_seed(20260005)
    a = (torch.rand(M, K, generator=g) * 2 - 1).to(torch.bfloat16)
    bt = (torch.rand(N, K, generator=g) * 2 - 1).to(torch.bfloat16)
    c = pkg.ops.gemm(a.to(gpu), bt.to(gpu), one_cta=one_cta)
    status = pkg.ops.sync_status()
    assert status == 0, pkg.native.strerror(status)
    assert c.dtype == torch.bfloat16 and tuple(c.shape) == (M, N)
    a_bits, bt_bits = bits(a), bits(bt)
    for bi, bj in _c5_blocks(7, 20260005):
        r0, c0 = bi * 256, bj * 256
        ref = oracle_mod.gemm_ref_c(a_bits[r0:r0 + 256], bt_bits[c0:c0 + 256])
        got = c[r0:r0 + 256, c0:c0 + 256].float().cpu().numpy()
        # one bf16 rounding of the fp32 sum (entries of C are of order sqrt(K) / 3)
        np.testing.assert_allclose(got, ref, rtol=2 ** -7, atol=2e-3, err_msg=f"block {bi},{bj}")
    # every element finite, and the whole of C has the spread the inputs imply
    assert torch.isfinite(c).all()
    assert 25.0 < float(c.float().std()) < 35.0
