"""Host-side properties of the library under concurrency, through the C ABI: launches
from several host threads on several streams give the results of serial launches, the
per-stream scratch table recycles its entries safely, and every stream has a status word
of its own."""
import threading

import pytest
import torch

from util import seeded_qkv

pytestmark = pytest.mark.gpu


def test_two_threads_two_streams_match_serial(pkg, gpu):
    """Attention and K-split GEMM launches issued concurrently by two host threads, each on
    its own stream, are bit-identical to the same launches made one after the other."""
    g = torch.Generator().manual_seed(321)
    q, k, v = (t.to(gpu) for t in seeded_qkv(1, 6, 640, 128, 55, 1.0))
    a = (torch.randn(256, 8192, generator=g) * 0.1).to(torch.bfloat16).to(gpu)
    bts = [(torch.randn(512, 8192, generator=g) * 0.1).to(torch.bfloat16).to(gpu) for _ in range(2)]
    want_o = [pkg.ops.fa_fwd(q, k, v, causal=c) for c in (False, True)]
    want_c = [pkg.ops.gemm(a, bt, f32_out=True) for bt in bts]
    assert pkg.ops.sync_status() == 0
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    outs_o = [torch.empty_like(want_o[0]) for _ in range(2)]
    outs_c = [torch.empty_like(want_c[0]) for _ in range(2)]
    errors = []

    def worker(i):
        try:
            torch.cuda.set_device(gpu)
            for _ in range(25):
                pkg.ops.fa_fwd(q, k, v, causal=bool(i), out=outs_o[i], stream=streams[i])
                pkg.ops.gemm(a, bts[i], out=outs_c[i], f32_out=True, stream=streams[i])
        except Exception as e:   # surfaced in the main thread
            errors.append(e)

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for i in range(2):
        assert pkg.ops.sync_status(streams[i]) == 0
        assert torch.equal(outs_o[i], want_o[i])
        assert torch.equal(outs_c[i], want_c[i])


def test_scratch_table_recycles_beyond_its_capacity(pkg, gpu):
    """More streams than the scratch table has entries (16): the least recently used
    buffer is waited for and recycled, results stay those of the first launch."""
    g = torch.Generator().manual_seed(99)
    a = (torch.randn(128, 4096, generator=g) * 0.1).to(torch.bfloat16).to(gpu)
    bt = (torch.randn(256, 4096, generator=g) * 0.1).to(torch.bfloat16).to(gpu)
    want = pkg.ops.gemm(a, bt, f32_out=True)
    free_before = None
    streams = [torch.cuda.Stream() for _ in range(40)]
    outs = [torch.empty_like(want) for _ in streams]
    for rnd in range(2):
        for st, o in zip(streams, outs):
            pkg.ops.gemm(a, bt, out=o, f32_out=True, stream=st)
        torch.cuda.synchronize()
        free = torch.cuda.mem_get_info()[0]
        if free_before is None:
            free_before = free
        # a second pass over 40 streams holds no more memory than the first
        assert free >= free_before - (8 << 20)
    assert pkg.ops.sync_status() == 0
    for o in outs:
        assert torch.equal(o, want)


def test_status_word_is_per_stream(pkg, gpu):
    """A wait that runs out on one stream (the probe's barrier that nobody arrives on)
    is reported on that stream only; the device-wide read sees it too and clears it."""
    s_bad, s_good = torch.cuda.Stream(), torch.cuda.Stream()
    q, k, v = (t.to(gpu) for t in seeded_qkv(1, 1, 256, 64, 3, 1.0))
    with torch.cuda.stream(s_good):
        pkg.ops.fa_fwd(q, k, v, stream=s_good)
    with torch.cuda.stream(s_bad):
        out, _ = pkg.ops.selftest(3)
    assert pkg.ops.sync_status(s_good) == 0
    code = pkg.ops.sync_status(s_bad)
    assert code > 0 and "probe" in pkg.native.strerror(code)
    assert pkg.ops.sync_status(s_bad) == 0          # consumed by the read
    with torch.cuda.stream(s_bad):
        pkg.ops.selftest(3)
    code = pkg.ops.sync_status()                    # device-wide
    assert code > 0 and "probe" in pkg.native.strerror(code)
    assert pkg.ops.sync_status() == 0 and pkg.ops.sync_status(s_bad) == 0
