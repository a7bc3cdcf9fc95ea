"""CPU tests of the multi-rank host logic: batch sharding and the slow-weight gradient
bucket with a world-size-2 gloo group."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from srwm_b200.dist import GradBucket, shard_range


def test_shard_range_covers_batch_exactly():
    for B in (1, 7, 8, 1024, 513):
        for n in (1, 2, 4, 8):
            spans = [shard_range(B, n, r) for r in range(n)]
            assert spans[0][0] == 0 and spans[-1][1] == B
            for (a, b), (c, d) in zip(spans, spans[1:]):
                assert b == c
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)


def test_bucket_layout_is_16_byte_aligned():
    b = GradBucket([(4, 16, 16), (4, 16, 4), (3, 5)], "cpu")
    for off, n in b.offsets:
        assert off % 4 == 0
    b.reduce_into(2, torch.ones(6, 3, 5))
    assert torch.equal(b.view(2), torch.full((3, 5), 6.0))
    b.reduce_into(2, torch.ones(2, 3, 5), accumulate=True)
    assert torch.equal(b.view(2), torch.full((3, 5), 8.0))
    assert b.all_reduce() is None          # no process group: no-op


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, H, E = 6, 2, 8
        g = torch.Generator().manual_seed(5)
        per_sample = [torch.randn(B, H, E, E, generator=g), torch.randn(B, H, E, 4, generator=g)]
        lo, hi = shard_range(B, world, rank)
        bucket = GradBucket([(H, E, E), (H, E, 4)], "cpu")
        for i, t in enumerate(per_sample):
            bucket.reduce_into(i, t[lo:hi])
        bucket.all_reduce()
        bucket.wait()
        ok = all(torch.allclose(bucket.view(i), t.sum(0), atol=1e-5) for i, t in enumerate(per_sample))
        # the training step's pattern: asynchronous all-reduce, overlapped with other work, waited
        # for before the bucket is written again
        for step in range(2):
            bucket.wait()
            for i, t in enumerate(per_sample):
                bucket.reduce_into(i, (step + 1) * t[lo:hi])
            work = bucket.all_reduce(async_op=True)
            ok = ok and work is not None
            _ = torch.randn(64, 64) @ torch.randn(64, 64)      # "the next forward"
        bucket.wait()
        ok = ok and bucket.work is None
        ok = ok and all(torch.allclose(bucket.view(i), 2 * t.sum(0), atol=1e-5) for i, t in enumerate(per_sample))
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


def test_bucket_allreduce_world_size_2_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, True), (1, True)]
