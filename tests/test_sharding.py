"""Multi-rank host logic on CPU: partitions are disjoint and exhaustive, and a
world_size-2 gloo run reproduces the single-rank result of the sharded path
(the per-shard compute is stood in for by the CPU oracle, since no GPU is
present here; the partitioning and the verification gather are what is tested)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_ranges_partition_everything(pkg):
    sh = pkg.sharding
    for total in (1, 7, 64, 256, 1000):
        for world in (1, 2, 3, 4, 8):
            parts = sh.all_shards(total, world)
            assert parts[0][0] == 0 and parts[-1][1] == total
            for (b0, e0), (b1, e1) in zip(parts, parts[1:]):
                assert e0 == b1 and e0 >= b0
            sizes = [e - b for b, e in parts]
            assert max(sizes) - min(sizes) <= 1
    assert sh.attention_shard(4, 16, 3, 8) == (24, 32)
    assert sh.gemm_column_shard(8192, 7, 8) == (7168, 8192)
    assert sh.row_shard(65537, 0, 8) == (0, 8193) and sh.row_shard(65537, 7, 8) == (57345, 65537)
    with pytest.raises(ValueError):
        sh.gemm_column_shard(100, 0, 2)
    with pytest.raises(ValueError):
        sh.shard_range(10, 2, 2)


def _worker(rank, world, port, tmpdir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import __graft_entry__ as ge
    import oracle
    pkg = ge.load_package()
    dist.init_process_group("gloo", rank=rank, world_size=world)
    B, H, S, D = 2, 3, 128, 32
    g = torch.Generator().manual_seed(2024)
    q, k, v = (torch.randn(B * H, S, D, generator=g).numpy() for _ in range(3))
    qb, kb, vb = (oracle.to_bf16_bits(x) for x in (q, k, v))
    b, e = pkg.sharding.attention_shard(B, H, rank, world)
    o_local = oracle.attention_ref_c(qb[b:e], kb[b:e], vb[b:e], 0.2, True, nthreads=1)
    s, a = pkg.sharding.gather_checksums(float(o_local.sum()), float(np.abs(o_local).sum()), dist)
    # gather the shards on rank 0 (verification gather)
    parts = [None] * world
    dist.all_gather_object(parts, (b, e, o_local))
    if rank == 0:
        full = np.concatenate([p[2] for p in sorted(parts, key=lambda t: t[0])])
        ref = oracle.attention_ref_c(qb, kb, vb, 0.2, True, nthreads=1)
        np.save(os.path.join(tmpdir, "ok.npy"), np.array([np.array_equal(full, ref),
                                                          abs(s - float(ref.sum())) < 1e-3,
                                                          abs(a - float(np.abs(ref).sum())) < 1e-3]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_sharded_attention(tmp_path):
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    ok = np.load(tmp_path / "ok.npy")
    assert ok.all()
