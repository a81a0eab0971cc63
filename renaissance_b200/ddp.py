"""Bucketed gradient mean all-reduce, overlapped with backward.

The reference reduces two fixed region ranges with one in-place FP32 ncclAllReduce
each and scales by 1/world afterwards (src/backend/ops/range/allreduce_op.cpp:37-105,
buckets at src/graph/compiler.cpp:1836-1847); only the first is overlapped with
compute.  Here the flat float gradient buffer is laid out in the order in which
backward completes its parameters and is cut into buckets (25 MB unless the caller
says otherwise; the VGG16-BN driver uses 50 MB); a bucket is cast half -> float (the reference's RANGE_CAST_FP16_TO_FP32, with the 1/world of the mean
folded in) and handed to NCCL as soon as backward has passed its end, so the
collective runs under the remaining backward kernels.  The wire format stays FP32
and the reduction is NCCL's (NVLink / NVSwitch), as in the reference.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def plan_buckets(total_elems: int, bucket_bytes: float, elem_bytes: int = 4):
    """[(begin, end)) element ranges of at most bucket_bytes, covering [0, total_elems)."""
    per = max(int(bucket_bytes // elem_bytes), 1)
    return [(a, min(a + per, total_elems)) for a in range(0, total_elems, per)]


class GradientBuckets:
    """g16: flat half gradients of the first `half_numel` elements; g32: flat float gradients of
    everything (elements past half_numel are produced in float directly).  `cast` converts a half
    range into the float buffer times a factor; `scale` scales a float range in place."""

    def __init__(self, g16, g32, half_numel, bucket_bytes=25 * 1024 * 1024, group=None, cast=None, scale=None):
        self.g16, self.g32, self.half_numel = g16, g32, int(half_numel)
        self.group = group
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.buckets = plan_buckets(g32.numel(), bucket_bytes)
        self.cast = cast or (lambda src, dst, factor: dst.copy_(src.float().mul_(factor)))
        self.scale = scale or (lambda t, factor: t.mul_(factor))
        self.next = 0
        self.works = []
        self.issued = []
        # "overlap": a bucket is all-reduced as soon as backward has passed it (the product's schedule);
        # "after": every bucket only once backward has finished; "skip": no all-reduce at all.  The last two exist
        # for the benchmark's diagnostics of what the collective costs.
        self.mode = "overlap"

    def begin_step(self):
        self.next = 0
        self.works = []
        self.issued = []

    def mark_ready(self, upto: int, final: bool = False):
        """Backward has produced every half gradient below element `upto`."""
        inv = 1.0 / self.world
        if self.mode == "after" and not final:
            return
        if final and self.world > 1 and self.half_numel < self.g32.numel():
            self.scale(self.g32[self.half_numel:], inv)         # float-born gradients: mean folded in here
        while self.next < len(self.buckets):
            a, b = self.buckets[self.next]
            if b > upto and not final:
                break
            hi = min(b, self.half_numel)
            if a < hi:
                self.cast(self.g16[a:hi], self.g32[a:hi], inv)
            if self.world > 1 and self.mode != "skip":
                self.works.append(dist.all_reduce(self.g32[a:b], op=dist.ReduceOp.SUM, group=self.group,
                                                  async_op=True))
            self.issued.append((a, b))
            self.next += 1

    def finish(self):
        self.mark_ready(self.g32.numel(), final=True)
        for w in self.works:
            w.wait()
        self.works = []
