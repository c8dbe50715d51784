"""fa_fwd_bf16_noalloc and fa_fwd_bf16_noalloc_status, through the C ABI.

fa_fwd_bf16_noalloc is for callers that must not trigger a device allocation
when they launch attention (a serving loop with all memory pre-carved, a
latency-critical section, a host runtime that owns the device pool): its scratch sits in
a static device array instead of the workspace that fa_fwd_bf16 cudaMalloc's on
first use. Both entry points run the same kernel code, so their outputs must be
identical; the test calls the new one twice in a row, because every call reuses
the same array and has to clear what the previous call left there. The status
read-back that belongs to it must report 0 after healthy launches.

This file sorts last on purpose: a run that stops at the first failure has then
already run every other test. It passes alone in a fresh process too (the new
entry point does its own per-device set-up on first use).
"""
import ctypes
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest
import torch

from util import ATTN_MAX_ABS, ATTN_MEAN_ABS, attn_errors, bits, seeded_qkv

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _call_noalloc(pkg, o, q, k, v, causal, flags=0):
    B, H, S, D = q.shape
    return pkg.native.lib().fa_fwd_bf16_noalloc(
        o.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), B, H, S, D,
        ctypes.c_float(1.0 / D ** 0.5), int(causal), flags, torch.cuda.current_stream().cuda_stream)


def _status(pkg, n_flags=240):
    flags = (ctypes.c_uint32 * max(n_flags, 1))()
    rc = pkg.native.lib().fa_fwd_bf16_noalloc_status(flags if n_flags else None, n_flags,
                                                     torch.cuda.current_stream().cuda_stream)
    return rc, list(flags)[:n_flags]


@pytest.mark.parametrize("D,causal", [(128, False), (128, True), (64, False), (64, True)])
def test_noalloc_matches_regular_entry_point_twice(pkg, gpu, D, causal):
    B, H, S = 2, 40, 768           # more work items than SMs: every CTA loops over several
    q, k, v = (t.to(gpu) for t in seeded_qkv(B, H, S, D, 31 + D, 1.0))
    # (the sibling call with its last round left uncut, as this entry point always leaves it)
    want = pkg.ops.fa_fwd(q, k, v, causal=causal, flags=pkg.native.FA_NO_TAIL_SPLIT)
    assert pkg.ops.sync_status() == 0
    for attempt in range(2):       # two calls in a row share the static scratch
        got = torch.full_like(want, float("nan"))
        rc = _call_noalloc(pkg, got, q, k, v, causal)
        assert rc == 0, pkg.native.strerror(rc)
        torch.cuda.synchronize()
        # same kernel code, same inputs: bit-identical (well inside the 2e-2 / 2e-3
        # tolerance the parity tests use against the oracle)
        assert torch.equal(got, want), f"call {attempt}"
        # the scratch can be read: no wait ran out, no CTA flagged
        code, cta_flags = _status(pkg)
        assert code == 0, pkg.native.strerror(code)
        assert not any(cta_flags)
    # different inputs right after: nothing stale is picked up from the scratch
    q2, k2, v2 = (t.to(gpu) for t in seeded_qkv(B, H, S, D, 977, 2.0))
    want2 = pkg.ops.fa_fwd(q2, k2, v2, causal=causal, flags=pkg.native.FA_NO_TAIL_SPLIT)
    got2 = torch.empty_like(want2)
    assert _call_noalloc(pkg, got2, q2, k2, v2, causal) == 0
    torch.cuda.synchronize()
    assert torch.equal(got2, want2)
    assert _status(pkg, 0)[0] == 0     # flags are optional


def test_noalloc_ragged_causal_against_the_oracle(pkg, gpu, oracle_mod):
    """A causal sequence length that is not a multiple of 128 is inside this entry
    point's contract; checked against the CPU oracle rather than the sibling call."""
    B, H, S, D = 1, 3, 300, 128
    q, k, v = seeded_qkv(B, H, S, D, 4242, 1.0)
    got = torch.full((B, H, S, D), float("nan"), dtype=torch.bfloat16, device=gpu)
    rc = _call_noalloc(pkg, got, q.to(gpu), k.to(gpu), v.to(gpu), True)
    assert rc == 0, pkg.native.strerror(rc)
    assert _status(pkg)[0] == 0
    ref = oracle_mod.attention_ref_c(*(bits(t).reshape(B * H, S, D) for t in (q, k, v)), 1.0 / D ** 0.5, True)
    mx, mean = attn_errors(got, ref)
    assert mx <= ATTN_MAX_ABS and mean <= ATTN_MEAN_ABS


def test_noalloc_rejects_bad_arguments(pkg, gpu):
    t = torch.zeros(1, 1, 256, 128, dtype=torch.bfloat16, device=gpu)
    L, n, P = pkg.native.lib(), pkg.native, t.data_ptr()
    sc = ctypes.c_float(0.1)
    assert L.fa_fwd_bf16_noalloc(P, P, P, P, 1, 1, 256, 96, sc, 0, 0, None) == n.E_SHAPE
    assert L.fa_fwd_bf16_noalloc(None, P, P, P, 1, 1, 256, 128, sc, 0, 0, None) == n.E_INVALID
    assert L.fa_fwd_bf16_noalloc(P, P + 2, P, P, 1, 1, 256, 128, sc, 0, 0, None) == n.E_ALIGN
    # documented limit: a non-causal sequence length must be a multiple of 128 here
    assert L.fa_fwd_bf16_noalloc(P, P, P, P, 1, 1, 300, 128, sc, 0, 0, None) == n.E_SHAPE
    # the capacity code has its own text
    assert b"capacity" in L.ptxb200_strerror(n.E_CAPACITY)
    assert L.fa_fwd_bf16_noalloc_status(None, 8, None) == n.E_INVALID
    assert L.fa_fwd_bf16_noalloc_status(None, -1, None) == n.E_INVALID


_FRESH = textwrap.dedent("""
    import ctypes, sys
    sys.path.insert(0, {root!r})
    import numpy as np, torch
    import __graft_entry__ as ge
    import oracle
    pkg = ge.load_package()
    L = pkg.native.lib()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    def qkv(B, H, S, D, seed):
        g = torch.Generator().manual_seed(seed)
        return [torch.randn(B, H, S, D, generator=g).to(torch.bfloat16) for _ in range(3)]
    cases = [(1, 2, 256, 128, 0), (2, 3, 384, 64, 1), (1, 4, 512, 64, 0), (1, 2, 300, 128, 1)]
    host = [qkv(B, H, S, D, 100 + i) for i, (B, H, S, D, c) in enumerate(cases)]
    devt = [[t.to(dev) for t in h] for h in host]
    outs = [torch.empty_like(d[0]) for d in devt]
    def call(i):
        B, H, S, D, causal = cases[i]
        q, k, v = devt[i]
        rc = L.fa_fwd_bf16_noalloc(outs[i].data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), B, H, S, D,
                                   ctypes.c_float(1.0 / D ** 0.5), causal, 0, None)
        assert rc == 0, rc
    # first use of each kernel variant loads its code (and torch's fill kernel, used below,
    # loads with its own first call); nothing else of this library has run
    for i in range(len(cases)):
        outs[i].fill_(float("nan"))
        call(i)
    assert L.fa_fwd_bf16_noalloc_status(None, 0, None) == 0
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    for rep in range(3):
        for i in range(len(cases)):
            outs[i].fill_(float("nan"))
            call(i)
        assert L.fa_fwd_bf16_noalloc_status(None, 0, None) == 0
    torch.cuda.synchronize()
    free1 = torch.cuda.mem_get_info()[0]
    assert free1 == free0, (free0, free1)
    oracle.build_c_oracle()
    for i, (B, H, S, D, causal) in enumerate(cases):
        b = [t.view(torch.int16).numpy().view(np.uint16).reshape(B * H, S, D) for t in host[i]]
        ref = oracle.attention_ref_c(*b, 1.0 / D ** 0.5, bool(causal))
        err = np.abs(outs[i].float().cpu().numpy().reshape(ref.shape) - ref)
        assert err.max() <= {max_abs} and err.mean() <= {mean_abs}, (i, err.max(), err.mean())
    print("FRESH-OK")
""")


def test_noalloc_in_a_fresh_process_leaves_free_memory_unchanged(gpu):
    """In a process where no other entry point of the library has run (so its workspace
    was never allocated), repeated fa_fwd_bf16_noalloc calls of several shapes leave the
    device's free memory exactly where it was, and their outputs match the CPU oracle."""
    code = _FRESH.format(root=ROOT, max_abs=ATTN_MAX_ABS, mean_abs=ATTN_MEAN_ABS)
    r = subprocess.run([sys.executable, "-c", code], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                       text=True, timeout=600)
    assert r.returncode == 0 and "FRESH-OK" in r.stdout, r.stdout[-3000:]
