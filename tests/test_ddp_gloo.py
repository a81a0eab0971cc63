"""World-size-2 checks of the data-parallel gradient path on CPU (gloo): the bucket
planner, the order in which buckets are handed to the collective, and the mean
all-reduce semantics the reference pins in tests/correction/test_mean_allreduce.cpp
(rank k fills its buffer with k; every rank must end with (N-1)/2)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from renaissance_b200.ddp import GradientBuckets, plan_buckets, plan_buckets_at


def test_plan_buckets_covers_range_once():
    b = plan_buckets(1000, 4 * 300)
    assert b == [(0, 300), (300, 600), (600, 900), (900, 1000)]
    assert plan_buckets(10, 1 << 20) == [(0, 10)]
    assert plan_buckets(0, 64) == []
    # VGG16-BN: 138.4 M parameters in 25 MB float buckets
    big = plan_buckets(138_365_992, 25 * 1024 * 1024)
    assert len(big) == 22 and big[-1][1] == 138_365_992 and all(e - s <= 6_553_600 for s, e in big)


def test_plan_buckets_at_tensor_ends():
    # buckets end only at the cuts, as soon as they hold the size asked for; the rest is the final bucket
    assert plan_buckets_at([100, 150, 1000, 1040, 1100], 1200, 4 * 120) == [(0, 150), (150, 1000), (1000, 1200)]
    assert plan_buckets_at([100, 200], 200, 4 * 1000) == [(0, 200)]
    assert plan_buckets_at([], 50, 4) == [(0, 50)]
    assert plan_buckets_at([10, 20, 30], 30, 4 * 10) == [(0, 10), (10, 20), (20, 30)]
    g32 = torch.zeros(1200)
    gb = GradientBuckets(torch.zeros(0, dtype=torch.float16), g32, 0, bucket_bytes=4 * 120, cuts=[100, 150, 1000])
    assert gb.buckets == [(0, 150), (150, 1000), (1000, 1200)]


def test_single_rank_is_cast_only():
    g16 = torch.arange(100, dtype=torch.float16)
    g32 = torch.full((130,), 5.0)
    gb = GradientBuckets(g16, g32, 100, bucket_bytes=4 * 32)
    gb.begin_step()
    gb.mark_ready(40)
    assert gb.issued == [(0, 32)]                      # only buckets that end below the mark
    gb.mark_ready(100)
    assert gb.issued == [(0, 32), (32, 64), (64, 96)]
    gb.finish()
    assert gb.issued[-1] == (128, 130) and len(gb.issued) == 5
    assert torch.equal(g32[:100], g16.float()) and bool((g32[100:] == 5.0).all())


def test_single_rank_float_born_head():
    h16 = torch.arange(40, dtype=torch.float16)
    g32 = torch.full((130,), 5.0)
    gb = GradientBuckets(h16, g32, 100, bucket_bytes=4 * 32, half_begin=60)
    gb.begin_step()
    gb.mark_ready(60)
    assert gb.issued == [(0, 32)]
    gb.mark_ready(100)
    assert gb.issued == [(0, 32), (32, 64), (64, 96)]
    gb.finish()
    assert len(gb.issued) == 5
    assert torch.equal(g32[60:100], h16.float()) and bool((g32[:60] == 5.0).all()) and bool((g32[100:] == 5.0).all())


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from renaissance_b200 import ops
        # (1) the reference's mean all-reduce test
        t = torch.full((1000,), float(rank))
        ops.mean_allreduce(t)
        ok_mean = bool(torch.allclose(t, torch.full((1000,), (world - 1) / 2.0), atol=1e-7))
        # (2) bucketed path: half gradients for the first 700 elements, float-born for the last 60
        gen = torch.Generator().manual_seed(rank)
        g16 = torch.randn(700, generator=gen).half()
        g32 = torch.zeros(760)
        g32[700:] = torch.randn(60, generator=gen)
        gb = GradientBuckets(g16, g32, 700, bucket_bytes=4 * 256)
        gb.begin_step()
        for mark in (100, 300, 512, 700):
            gb.mark_ready(mark)
        issued_before_finish = list(gb.issued)
        gb.finish()
        # expected mean over ranks, computed by every rank from the seeds
        exp = torch.zeros(760)
        for r in range(world):
            gr = torch.Generator().manual_seed(r)
            h = torch.randn(700, generator=gr).half().float()
            f = torch.randn(60, generator=gr)
            exp[:700] += h / world
            exp[700:] += f / world
        ok_bucket = bool(torch.allclose(g32, exp, atol=1e-6))
        # (3) the VGG16-BN driver's layout: float-born gradients first (the FC weights), then the half range, then
        # float-born vectors; the half buffer holds the middle range only
        gen = torch.Generator().manual_seed(10 + rank)
        f32 = torch.randn(900, generator=gen)
        h16 = torch.randn(400, generator=gen).half()
        g32 = f32.clone()
        gb = GradientBuckets(h16, g32, 700, bucket_bytes=4 * 256, half_begin=300)
        gb.begin_step()
        gb.mark_ready(300)               # the float-born head is complete: one whole bucket lies inside it
        head_only = list(gb.issued)
        gb.mark_ready(700)
        gb.finish()
        exp = torch.zeros(900)
        for r in range(world):
            gr = torch.Generator().manual_seed(10 + r)
            f = torch.randn(900, generator=gr)
            h = torch.randn(400, generator=gr).half().float()
            f[300:700] = h
            exp += f / world
        ok_bucket = ok_bucket and bool(torch.allclose(g32, exp, atol=1e-6)) and head_only == [(0, 256)] \
            and list(gb.issued) == [(0, 256), (256, 512), (512, 768), (768, 900)]
        results[rank] = (ok_mean, ok_bucket, issued_before_finish, list(gb.issued))
    finally:
        dist.destroy_process_group()


def test_two_ranks_gloo():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert len(results) == world
    for rank in range(world):
        ok_mean, ok_bucket, before, after = results[rank]
        assert ok_mean and ok_bucket
        assert before == [(0, 256), (256, 512)]
        assert after == [(0, 256), (256, 512), (512, 768), (768, 900)]
