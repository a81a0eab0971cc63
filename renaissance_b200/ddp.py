"""Bucketed gradient mean all-reduce, overlapped with backward.

The reference reduces two fixed region ranges with one in-place FP32 ncclAllReduce
each and scales by 1/world afterwards (src/backend/ops/range/allreduce_op.cpp:37-105,
buckets at src/graph/compiler.cpp:1836-1847); only the first is overlapped with
compute.  Here the flat float gradient buffer is laid out in the order in which
backward completes its parameters and is cut into buckets (equal ones of 25 MB unless
the caller says otherwise; the VGG16-BN driver ends them at tensor ends, 50 MB or more
each); a bucket's half gradients are
cast half -> float (the reference's RANGE_CAST_FP16_TO_FP32) and the bucket is handed
to NCCL as soon as backward has passed its end, so the collective runs under the
remaining backward kernels.  The wire format stays FP32 and the reduction is NCCL's
(NVLink / NVSwitch), as in the reference.  The 1/world of the mean is NCCL's own
(ncclAvg) where the backend has it; otherwise it is folded into the cast, and the
gradients born in float (the reference's FC_AMP_BWD writes dW in float,
fc_op.cpp:434-446; BN vectors; biases) are scaled in place before their bucket goes out.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def plan_buckets(total_elems: int, bucket_bytes: float, elem_bytes: int = 4):
    """[(begin, end)) element ranges of at most bucket_bytes, covering [0, total_elems)."""
    per = max(int(bucket_bytes // elem_bytes), 1)
    return [(a, min(a + per, total_elems)) for a in range(0, total_elems, per)]


def plan_buckets_at(cuts, total_elems: int, bucket_bytes: float, elem_bytes: int = 4):
    """Buckets that end only at the given element offsets (ascending; the ends of the tensors backward completes one
    after the other), each closed as soon as it holds bucket_bytes: a tensor that becomes ready in one piece (the
    411 MB weight gradient of VGG16's first FC layer) goes out as one collective instead of many that all start at
    the same moment.  What follows the last cut is the final bucket."""
    out, a = [], 0
    for c in cuts:
        c = min(int(c), total_elems)
        if c > a and (c - a) * elem_bytes >= bucket_bytes:
            out.append((a, c))
            a = c
    if a < total_elems:
        out.append((a, total_elems))
    return out


class GradientBuckets:
    """g32: flat float gradients of everything.  Elements [half_begin, half_numel) are produced in half, in
    `g16` (whose element 0 is flat element half_begin); every other element is produced in float directly.
    `cast` converts a half range into the float buffer times a factor; `scale` scales a float range in place.
    `cuts`: element offsets at which a bucket may end (plan_buckets_at); None cuts equal buckets."""

    def __init__(self, g16, g32, half_numel, bucket_bytes=25 * 1024 * 1024, group=None, cast=None, scale=None,
                 half_begin=0, cuts=None):
        self.g16, self.g32 = g16, g32
        self.half_begin, self.half_numel = int(half_begin), int(half_numel)
        self.group = group
        live = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if live else 1
        # the mean: NCCL divides inside the collective; other backends (gloo) sum what was scaled beforehand
        self.native_mean = bool(live and self.world > 1 and dist.get_backend(group) == "nccl")
        self.buckets = plan_buckets(g32.numel(), bucket_bytes) if cuts is None else \
            plan_buckets_at(cuts, g32.numel(), bucket_bytes)
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
        """Backward has produced every gradient below element `upto` (`final`: every gradient)."""
        pre = 1.0 if (self.native_mean or self.world == 1) else 1.0 / self.world
        if self.mode == "after" and not final:
            return
        hb, he = self.half_begin, self.half_numel
        while self.next < len(self.buckets):
            a, b = self.buckets[self.next]
            if (b > upto or b > he) and not final:      # elements past the half range are complete only at the end
                break
            lo, hi = max(a, hb), min(b, he)
            if lo < hi:
                self.cast(self.g16[lo - hb:hi - hb], self.g32[lo:hi], pre)
            if pre != 1.0:
                for fa, fb in ((a, min(b, hb)), (max(a, he), b)):
                    if fa < fb:
                        self.scale(self.g32[fa:fb], pre)
            if self.world > 1 and self.mode != "skip":
                op = dist.ReduceOp.AVG if self.native_mean else dist.ReduceOp.SUM
                self.works.append(dist.all_reduce(self.g32[a:b], op=op, group=self.group, async_op=True))
            self.issued.append((a, b))
            self.next += 1

    def finish(self):
        self.mark_ready(self.g32.numel(), final=True)
        for w in self.works:
            w.wait()
        self.works = []
