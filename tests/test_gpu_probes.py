"""Bring-up probes with known answers, through the C ABI (ptxb200_selftest).

Restates the reference's single-instruction runtime tests: TMEM round-trip
identity (test/gpu/blackwell/tcgen05_roundtrip.jl:78-88) and single-MMA known
answers (tcgen05_mma_probe.jl:122-129: ones x ones over K=16 -> 16.0), plus the
non-uniform operand forms the attention kernel depends on.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_tmem_roundtrip(pkg, gpu):
    out_s, _ = pkg.ops.selftest(0)
    assert pkg.ops.sync_status() == 0
    got = out_s.cpu().numpy().view(np.uint32)
    r = np.arange(128, dtype=np.uint32)[:, None]
    c = np.arange(128, dtype=np.uint32)[None, :]
    assert np.array_equal(got, ((r << 16) | c) ^ np.uint32(0x5A5A0000))


@pytest.mark.parametrize("which,D", [(1, 128), (2, 64)])
def test_tile_ones(pkg, gpu, which, D):
    """All-ones operands: S = D, O = 128 exactly (the reference's 16.0 probe, scaled)."""
    one = lambda *s: torch.ones(*s, dtype=torch.bfloat16, device=gpu)
    out_s, out_o = pkg.ops.selftest(which, one(128, D), one(128, D), one(128, D), one(128, 128))
    assert pkg.ops.sync_status() == 0
    assert torch.all(out_s == float(D))
    assert torch.all(out_o == 128.0)


@pytest.mark.parametrize("which,D", [(1, 128), (2, 64)])
def test_tile_random(pkg, gpu, oracle_mod, which, D):
    """Non-uniform data: exercises the swizzled K-major descriptors, the MN-major V
    descriptor and P read from tensor memory. Products of bf16 values accumulate
    exactly enough in fp32 for a tight tolerance."""
    g = torch.Generator().manual_seed(77 + D)
    q, k, v = (torch.randn(128, D, generator=g).to(torch.bfloat16) for _ in range(3))
    p = torch.rand(128, 128, generator=g).to(torch.bfloat16)
    out_s, out_o = pkg.ops.selftest(which, q.to(gpu), k.to(gpu), v.to(gpu), p.to(gpu))
    assert pkg.ops.sync_status() == 0
    s_ref = q.float().numpy() @ k.float().numpy().T
    o_ref = p.float().numpy() @ v.float().numpy()
    np.testing.assert_allclose(out_s.cpu().numpy(), s_ref, rtol=1e-4, atol=1e-3)
    np.testing.assert_allclose(out_o.cpu().numpy(), o_ref, rtol=1e-4, atol=1e-3)


def test_bounded_wait_expiry_is_reported_and_the_device_stays_usable(pkg, gpu):
    """A wait that nothing satisfies gives up after its limit: the kernel returns, the
    status word names the wait site, a second wait in the CTA returns at once, and the
    library keeps working afterwards (no trap, no fault, no hang)."""
    import time
    assert pkg.ops.sync_status() == 0
    t0 = time.perf_counter()
    out, _ = pkg.ops.selftest(3)
    status = pkg.ops.sync_status()
    dt = time.perf_counter() - t0
    assert 1.0 < dt < 10.0                       # the 1.5 s wait limit, not a hang
    assert out.cpu().tolist()[:3] == [0, 0, 0xD0E5]
    assert status > 0 and (status >> 24) == 0x32 and ((status >> 8) & 0xFF) == 15
    assert "probe" in pkg.native.strerror(status)
    assert pkg.ops.sync_status() == 0             # reading the status cleared it
    test_tmem_roundtrip(pkg, gpu)                 # the device is as usable as before


def test_ex2_throughput_probe(pkg, gpu):
    """The exponential unit's throughput, the second bound of the attention kernel: at most
    16 ex2 per clock per SM however many warps issue them (a saturated pipe with 16 warps),
    and the softmax's inner mix stays within a fifth of that."""
    out, _ = pkg.ops.selftest(4)
    assert pkg.ops.sync_status() == 0
    v = out.cpu().tolist()
    rate = [v[2 * k + 1] / v[2 * k] for k in range(5)]
    assert all(r <= 16.6 for r in rate), rate
    assert rate[2] >= 14.0, rate          # 16 warps of pure ex2 saturate the pipe
    assert rate[4] >= 0.75 * rate[2], rate
