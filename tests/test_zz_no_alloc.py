"""fa_fwd_bf16_noalloc against fa_fwd_bf16, through the C ABI.

fa_fwd_bf16_noalloc is for callers that must not trigger a device allocation
when they launch attention (a serving loop with all memory pre-carved, a
latency-critical section, a host runtime that owns the device pool): its scratch sits in
a static device array instead of the workspace that fa_fwd_bf16 cudaMalloc's on
first use. Both entry points run the same kernel code, so their outputs must be
identical; the test calls the new one twice in a row, because every call reuses
the same array and has to clear what the previous call left there.

This file sorts last on purpose: a run that stops at the first failure has then
already run every other test. It passes alone in a fresh process too (the new
entry point does its own per-device set-up on first use).
"""
import ctypes

import pytest
import torch

from util import seeded_qkv

pytestmark = pytest.mark.gpu


def _call_noalloc(pkg, o, q, k, v, causal, flags=0):
    B, H, S, D = q.shape
    return pkg.native.lib().fa_fwd_bf16_noalloc(
        o.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), B, H, S, D,
        ctypes.c_float(1.0 / D ** 0.5), int(causal), flags, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("D,causal", [(128, False), (128, True), (64, False), (64, True)])
def test_noalloc_matches_regular_entry_point_twice(pkg, gpu, D, causal):
    B, H, S = 2, 40, 768           # more work items than SMs: every CTA loops over several
    q, k, v = (t.to(gpu) for t in seeded_qkv(B, H, S, D, 31 + D, 1.0))
    want = pkg.ops.fa_fwd(q, k, v, causal=causal)
    assert pkg.ops.sync_status() == 0
    for attempt in range(2):       # two calls in a row share the static scratch
        got = torch.full_like(want, float("nan"))
        rc = _call_noalloc(pkg, got, q, k, v, causal)
        assert rc == 0, pkg.native.strerror(rc)
        torch.cuda.synchronize()
        # same kernel code, same inputs: bit-identical (well inside the 2e-2 / 2e-3
        # tolerance the parity tests use against the oracle)
        assert torch.equal(got, want), f"call {attempt}"
    # different inputs right after: nothing stale is picked up from the scratch
    q2, k2, v2 = (t.to(gpu) for t in seeded_qkv(B, H, S, D, 977, 2.0))
    want2 = pkg.ops.fa_fwd(q2, k2, v2, causal=causal)
    got2 = torch.empty_like(want2)
    assert _call_noalloc(pkg, got2, q2, k2, v2, causal) == 0
    torch.cuda.synchronize()
    assert torch.equal(got2, want2)


def test_noalloc_rejects_bad_arguments(pkg, gpu):
    t = torch.zeros(1, 1, 256, 128, dtype=torch.bfloat16, device=gpu)
    L, n, P = pkg.native.lib(), pkg.native, t.data_ptr()
    sc = ctypes.c_float(0.1)
    assert L.fa_fwd_bf16_noalloc(P, P, P, P, 1, 1, 256, 96, sc, 0, 0, None) == n.E_SHAPE
    assert L.fa_fwd_bf16_noalloc(None, P, P, P, 1, 1, 256, 128, sc, 0, 0, None) == n.E_INVALID
    assert L.fa_fwd_bf16_noalloc(P, P + 2, P, P, 1, 1, 256, 128, sc, 0, 0, None) == n.E_ALIGN
