#!/usr/bin/env python3
"""VGG16-BN AMP training-step benchmark (BASELINE.json: "VGG16-BN fwd+bwd images/sec").

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the CPU restatement of the reference path, host cores

One step = forward + backward + gradient all-reduce + SGD-momentum of VGG16-BN on a
synthetic batch of 256 images per GPU (NHWC half, 224x224x3 padded to 4 channels,
N(0,1); labels uniform in 0..999; random-init weights), loss scale 1024, gradient
buckets of 50 MB or more that end at tensor ends.  Prints ONE JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "vgg16bn_fwd_bwd_images_per_sec"
UNIT = "images/s"
BATCH_PER_GPU = 256
IMAGE = 224
CLASSES = 1000

# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) over algorithmic bytes of
# conv3x3_igemm_kernel<256>, from the ncu capture in
# profiles/conv3x3_igemm_kernel_n256_fprop_stats_64x56x56x256.md (163.8 / 206.7 MB).  Full-size launches
# are too large to capture under --set full, and the traffic grows in proportion to the tensors, so the
# per-launch traffic reported below is the launches' average algorithmic byte count times this ratio.
ROOFLINE_TRAFFIC_RATIO = 0.79


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], tflops=p.get("bf16_tflops_sustained", p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in self.rows:
            parts = [p.strip() for p in row.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def conv_flops_per_step(batch):
    """2*N*H*W*K*9*C per pass; forward 13 layers (3 real input channels in the first), backward dgrad 12 + wgrad 13."""
    from renaissance_b200.vgg16bn import VGG16_CFG
    h, c, total = IMAGE, 3, 0.0
    first = True
    for v in VGG16_CFG:
        if v == "M":
            h //= 2
            continue
        f = 2.0 * batch * h * h * v * 9 * c
        total += f * (2 if first else 3)
        first = False
        c = v
    return total


def config2_block(peaks_burst_tflops, hbm_gbs, iters=7):
    """BASELINE.json configuration 2 beside the step: one Conv3x3(64 -> 64) + BN + ReLU block backward at batch 256,
    56 x 56, through trb200_cbr_bwd on its three streams; CUDA events, a 512 MB write between calls (L2 flushed),
    median.  ideal = the two convolutions' flop at the measured burst tensor peak (the block is timed alone) + the BN
    backward's 10.25 B/element at the measured copy bandwidth."""
    import torch
    from renaissance_b200 import ops
    n, h, c, k = 256, 56, 64, 64
    geo = ops.ConvGeometry(n, h, h, c, k)
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn((n, h, h, c), generator=g, device="cuda").half()
    w = (torch.randn((k, 3, 3, c), generator=g, device="cuda") * (2.0 / (9 * c)) ** 0.5).half()
    dy = torch.randn((n, h, h, k), generator=g, device="cuda").half()
    conv_out = torch.randn((n, h, h, k), generator=g, device="cuda").half()
    bits = torch.randint(0, 256, (n * h * h * k // 8,), generator=g, device="cuda", dtype=torch.int32).to(torch.uint8)
    gamma = torch.ones(k, device="cuda")
    mean = conv_out.float().mean(dim=(0, 1, 2))
    inv = 1.0 / torch.sqrt(conv_out.float().var(dim=(0, 1, 2), unbiased=False) + 1e-5)
    scratch = torch.empty_like(dy)
    dw = torch.empty_like(w)
    st = ops.BlockStreams.create()
    flush = torch.empty(512 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()

    def call():
        with torch.cuda.stream(st.bn):
            ops.cbr_amp_bwd(geo, dy, w, gamma, mean, inv, bits, x, conv_out, bn_scratch=scratch, dw=dw, streams=st)
        torch.cuda.current_stream().wait_stream(st.bn)

    torch.cuda.current_stream().wait_stream(st.bn)
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        call()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ops.device_status()
    med = statistics.median(ts)
    flop = 2 * 2.0 * n * h * h * c * k * 9
    byt = 10.25 * n * h * h * k
    ideal = flop / peaks_burst_tflops / 1e9 + byt / hbm_gbs / 1e6
    return dict(workload="Conv3x3 64->64 + BN + ReLU block backward, batch 256, 56x56, fp16", ms=round(med, 4),
                ideal_ms=round(ideal, 4), frac=round(ideal / med, 4),
                note="ideal = conv flop at the measured burst tensor peak + BN bytes at the measured copy bandwidth")


def run_ours(args):
    import torch
    import torch.distributed as dist

    from renaissance_b200 import ops
    from renaissance_b200.vgg16bn import Vgg16BnTrainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("bench.py --gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        opts = None
        if args.nccl_high_priority:
            opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), pg_options=opts)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    batch = args.batch
    tr = Vgg16BnTrainer(batch=batch, image=IMAGE, classes=CLASSES, loss_scale=1024.0, bucket_mb=args.bucket_mb,
                        seed=1234, nccl_registered=None if args.nccl_registered == "off" else args.nccl_registered,
                        bucket_plan=args.bucket_plan)
    # synthetic batches in pinned host memory (two, alternated): images ~ N(0,1), 4th channel zero
    gen = torch.Generator().manual_seed(100 + rank)
    host_images, host_labels = [], []
    for _ in range(2):
        img = torch.zeros((batch, IMAGE, IMAGE, 4), dtype=torch.float16).pin_memory()
        img[..., :3] = torch.randn((batch, IMAGE, IMAGE, 3), generator=gen).half()
        host_images.append(img)
        host_labels.append(torch.randint(0, CLASSES, (batch,), generator=gen, dtype=torch.int32).pin_memory())
    for s in range(2):
        tr.upload(s, host_images[s], host_labels[s])
    torch.cuda.current_stream().wait_stream(tr.copy_stream)
    torch.cuda.synchronize()

    # ---------------- device-resident timing: W warm-up steps, then exactly K timed steps
    for _ in range(args.warmup):
        tr.step(0)
    ops.device_status()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    tr.timing = []
    tr.timing_bwd = []
    launches0 = ops.kernel_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        loss = tr.step(i & 1)
    e1.record()
    barrier()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    launches = ops.kernel_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    roof_events = tr.timing
    bwd_events = tr.timing_bwd
    tr.timing = None
    tr.timing_bwd = None
    ops.device_status()
    loss_value = float(loss.item())
    ms_per_step = ms_total / args.steps
    value = world * batch * args.steps / (ms_total / 1e3)

    # ---------------- roofline of the dominant kernel (conv3x3_igemm_kernel<256>): its forward launches
    # (the nine layers with 256 or 512 filters), bracketed by CUDA events inside the timed region on the
    # launching stream; each bracket also holds the few-microsecond bn_stats_finalize launch that follows
    peaks = measured_peaks()
    flops = sum(e[2] for e in roof_events)
    dur_ms = sum(e[0].elapsed_time(e[1]) for e in roof_events)
    alg_bytes = sum(e[3] for e in roof_events)
    n_l = max(len(roof_events), 1)
    achieved = flops / (dur_ms / 1e3) / 1e12 if dur_ms > 0 else 0.0
    roofline = dict(kernel="conv3x3_igemm_kernel<256> (9 forward launches per step)", bound="tensor",
                    achieved=round(achieved, 1), peak=peaks["tflops"], unit="TFLOP/s",
                    frac=round(achieved / peaks["tflops"], 4), peak_source=peaks["source"],
                    flop_per_launch=flops / n_l, ms_per_launch=dur_ms / n_l, launches_timed=len(roof_events),
                    traffic=round(ROOFLINE_TRAFFIC_RATIO * alg_bytes / n_l),
                    traffic_note="average algorithmic bytes per launch x 0.79 (ncu DRAM/algorithmic ratio)")

    # ---------------- the named hot path inside the same timed region: every block backward's three stages, bracketed
    # by CUDA events that trb200_cbr_bwd records on the launching stream(s) before the BN stage and after the BN,
    # weight-gradient and data-gradient stages
    hot = dict(bn=[0.0, 0.0], wgrad=[0.0, 0.0], dgrad=[0.0, 0.0])      # [ms, bytes or flop]
    for L, ev in bwd_events:
        e_bn = L.k * batch * L.h * L.h
        hot["bn"][0] += ev[0].elapsed_time(ev[1])
        # two sweeps over dy (pooled: a quarter of it + the argmax byte), x, mask; one write of dconv
        hot["bn"][1] += (10.25 * e_bn if not L.pool_after else (2 * (2 + 0.125) + 2) * e_bn + 2 * (2 + 1) * e_bn / 4)
        hot["wgrad"][0] += ev[1].elapsed_time(ev[2])
        hot["wgrad"][1] += 2.0 * batch * L.h * L.h * L.k * 9 * (3 if L.idx == 0 else L.c)
        if L.idx > 0:
            hot["dgrad"][0] += ev[2].elapsed_time(ev[3])
            hot["dgrad"][1] += 2.0 * batch * L.h * L.h * L.k * 9 * L.c
    steps_f = float(args.steps)
    roofline_hot_path = dict(
        note="per step, summed over the 13 block backwards, CUDA events inside the timed region",
        bnrelu_bwd=dict(bound="hbm", ms=round(hot["bn"][0] / steps_f, 4), algorithmic_gb=round(hot["bn"][1] / steps_f / 1e9, 3),
                        achieved=round(hot["bn"][1] / (hot["bn"][0] / 1e3) / 1e9, 1), peak=peaks["hbm_gbs"], unit="GB/s",
                        frac=round(hot["bn"][1] / (hot["bn"][0] / 1e3) / 1e9 / peaks["hbm_gbs"], 4)),
        wgrad=dict(bound="tensor", ms=round(hot["wgrad"][0] / steps_f, 4), tflop=round(hot["wgrad"][1] / steps_f / 1e12, 3),
                   achieved=round(hot["wgrad"][1] / (hot["wgrad"][0] / 1e3) / 1e12, 1), peak=peaks["tflops"], unit="TFLOP/s",
                   frac=round(hot["wgrad"][1] / (hot["wgrad"][0] / 1e3) / 1e12 / peaks["tflops"], 4)),
        dgrad=dict(bound="tensor", ms=round(hot["dgrad"][0] / steps_f, 4), tflop=round(hot["dgrad"][1] / steps_f / 1e12, 3),
                   achieved=round(hot["dgrad"][1] / (hot["dgrad"][0] / 1e3) / 1e12, 1), peak=peaks["tflops"], unit="TFLOP/s",
                   frac=round(hot["dgrad"][1] / (hot["dgrad"][0] / 1e3) / 1e12 / peaks["tflops"], 4)),
        peak_source=peaks["source"])

    # ---------------- end to end: host buffers, H2D of every step's batch and D2H of its loss inside the region
    barrier()
    t0 = time.perf_counter()
    tr.upload(0, host_images[0], host_labels[0])
    for i in range(args.steps):
        s = i & 1
        if i + 1 < args.steps:
            tr.upload(s ^ 1, host_images[s ^ 1], host_labels[s ^ 1])      # prefetch the next batch (double buffer)
        l = tr.step(s, wait_copy=True)
        _ = float(l.item())                                                # device -> host read of the loss
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    h2d = host_images[0].numel() * 2 + host_labels[0].numel() * 4
    e2e = dict(value=round(world * batch * args.steps / e2e_s, 1), unit=UNIT, h2d_bytes_per_step=h2d,
               d2h_bytes_per_step=4)

    # ---------------- the device-resident region once more, after the end-to-end one: the two regions run under a
    # power-cap clock that drifts, so `value` and `e2e` are comparable only to the spread between these two
    barrier()
    r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    r0.record()
    for i in range(args.steps):
        tr.step(i & 1)
    r1.record()
    barrier()
    value_again = world * batch * args.steps / (max_over_ranks(r0.elapsed_time(r1)) / 1e3)

    # ---------------- multi-GPU diagnostics (outside the reported regions): where the all-reduce costs time
    comm = None
    if world > 1:
        def region(mode):
            tr.buckets.mode = mode
            for i in range(2):
                tr.step(i & 1)
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for i in range(args.steps):
                tr.step(i & 1)
            b.record()
            barrier()
            tr.buckets.mode = "overlap"
            return max_over_ranks(a.elapsed_time(b)) / args.steps
        ms_none = region("skip")          # no all-reduce at all: the step's compute alone (the ranks' weights drift apart)
        ms_after = region("after")        # every bucket all-reduced only after backward has finished: nothing overlaps
        tr.sync_weights_from_rank0()      # the skip region let the ranks drift: make them equal again
        comm = dict(step_ms_no_allreduce=round(ms_none, 3), step_ms_allreduce_after_backward=round(ms_after, 3),
                    comm_exposed_ms=round(ms_per_step - ms_none, 3),
                    comm_serial_ms=round(ms_after - ms_none, 3),
                    note="comm_exposed = overlapped step - step without all-reduce (what the overlap fails to hide, plus "
                         "what NCCL's CTAs take from the compute kernels); comm_serial = the all-reduce's own time")
        # ranks must hold identical master weights after identical updates of all-reduced gradients
        for i in range(2):
            tr.step(i & 1)
        barrier()
        chk = torch.stack([tr.w32.double().sum(), tr.w32.double().abs().sum()])
        lo, hi = chk.clone(), chk.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        if not bool(torch.equal(lo, hi)):
            raise SystemExit(f"rank {rank}: master weights differ between ranks after the all-reduced update "
                             f"(checksum min {lo.tolist()} max {hi.tolist()})")
        comm["weights_identical_on_all_ranks"] = True

    # ---------------- BASELINE configuration 2 (the single block backward) beside the step, single GPU run only
    block2 = None
    if rank == 0 and world == 1:
        burst = peaks["tflops"]
        path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(path):
            with open(path) as f:
                burst = json.load(f).get("bf16_tflops", burst)
        del tr
        torch.cuda.empty_cache()
        block2 = config2_block(burst, peaks["hbm_gbs"])

    # ---------------- CPU baseline beside it (rank 0, single GPU run only): the oracle's step on host cores
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(sample_batch=1)

    if rank == 0:
        line = dict(metric=METRIC, value=round(value, 1), unit=UNIT, n_gpus=world, steps=args.steps, warmup=args.warmup,
                    ms_per_step=round(ms_per_step, 3), higher_is_better=True, scaling="weak", vs_baseline=None,
                    dtype="fp16", data="synthetic",
                    config=dict(workload="VGG16-BN AMP fwd+bwd+allreduce+SGD-momentum, NHWC 224x224x3(+1 pad), "
                                         "batch 256/GPU, loss scale 1024, %g MB buckets (%s)" % (args.bucket_mb, args.bucket_plan),
                                global_batch=world * batch, parallelism=f"dp{world}",
                                l2="activations (>15 GB per step) far exceed the 126 MB L2; no flush needed",
                                conv_tflop_per_step_per_gpu=round(conv_flops_per_step(batch) / 1e12, 2),
                                loss=round(loss_value, 4)),
                    clocks=clocks, e2e=e2e, gpu_launches=int(launches // args.steps), roofline=roofline,
                    roofline_hot_path=roofline_hot_path, value_second_region=round(value_again, 1))
        if block2 is not None:
            line["roofline_hot_path"]["config2_block"] = block2
        if comm is not None:
            line["comm"] = comm
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_resnet50(args):
    """BASELINE.json configuration 4 (ResNet-50, bfloat16, batch 256 per GPU, bucketed all-reduce overlapped with
    backward) through renaissance_b200/resnet50.py.  Not the headline metric: the reference has no backend for this
    network, so there is no reference arm and no CPU baseline for it; the line carries the same timing rules."""
    import torch
    import torch.distributed as dist

    from renaissance_b200 import ops
    from renaissance_b200 import resnet50 as R

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world == 1 and args.gpus > 1:
        raise SystemExit("bench.py --gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    batch = args.batch
    dtype = torch.bfloat16
    net = R.ResNet50(dtype=dtype, seed=1234)                   # same seed: the ranks start from the same weights
    gen = torch.Generator().manual_seed(100 + rank)
    host_images, host_labels, dev_images, dev_labels = [], [], [], []
    for _ in range(2):
        img = torch.zeros((batch, IMAGE, IMAGE, 4), dtype=dtype).pin_memory()
        img[..., :3] = torch.randn((batch, IMAGE, IMAGE, 3), generator=gen).to(dtype)
        host_images.append(img)
        host_labels.append(torch.randint(0, CLASSES, (batch,), generator=gen, dtype=torch.int32).pin_memory())
        dev_images.append(img.cuda())
        dev_labels.append(host_labels[-1].cuda())
    copy_stream = torch.cuda.Stream()

    for i in range(args.warmup):
        net.step(dev_images[i & 1], dev_labels[i & 1])
    ops.device_status()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    net.timing_bn = []
    launches0 = ops.kernel_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        loss = net.step(dev_images[i & 1], dev_labels[i & 1])
    e1.record()
    barrier()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    launches = ops.kernel_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    bn_events = net.timing_bn
    net.timing_bn = None
    ops.device_status()
    ms_per_step = ms_total / args.steps
    value = world * batch * args.steps / (ms_total / 1e3)

    # the dominant kernels of this network are the BN backward sweeps (HBM-bound): 53 launches groups per step,
    # bracketed by CUDA events inside the timed region; 10.25 B per element with a ReLU mask, 10 without
    peaks = measured_peaks()
    bn_ms = sum(ev[0].elapsed_time(ev[1]) for ev, _, _ in bn_events)
    bn_bytes = sum((10.25 if masked else 10.0) * elems for _, elems, masked in bn_events)
    n_l = max(len(bn_events), 1)
    achieved = bn_bytes / (bn_ms / 1e3) / 1e9 if bn_ms > 0 else 0.0
    roofline = dict(kernel="bnrelu_bwd (reduce + finalize + apply; 53 per step)", bound="hbm", achieved=round(achieved, 1),
                    peak=peaks["hbm_gbs"], unit="GB/s", frac=round(achieved / peaks["hbm_gbs"], 4),
                    peak_source=peaks["source"], bytes_per_launch=bn_bytes / n_l, ms_per_launch=bn_ms / n_l,
                    launches_timed=len(bn_events), traffic=None)

    # end to end: the step's batch copied from pinned host memory (double buffered), the loss read back every step
    barrier()
    t0 = time.perf_counter()
    done = [torch.cuda.Event(), torch.cuda.Event()]
    with torch.cuda.stream(copy_stream):
        dev_images[0].copy_(host_images[0], non_blocking=True)
        dev_labels[0].copy_(host_labels[0], non_blocking=True)
        done[0].record()
    for i in range(args.steps):
        sl = i & 1
        if i + 1 < args.steps:
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_stream(torch.cuda.current_stream())      # the slot's previous step has finished with it
                dev_images[sl ^ 1].copy_(host_images[sl ^ 1], non_blocking=True)
                dev_labels[sl ^ 1].copy_(host_labels[sl ^ 1], non_blocking=True)
                done[sl ^ 1].record()
        torch.cuda.current_stream().wait_event(done[sl])
        l = net.step(dev_images[sl], dev_labels[sl])
        _ = float(l.item())
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    h2d = host_images[0].numel() * 2 + host_labels[0].numel() * 4
    e2e = dict(value=round(world * batch * args.steps / e2e_s, 1), unit=UNIT, h2d_bytes_per_step=h2d, d2h_bytes_per_step=4)

    identical = None
    if world > 1:
        chk = torch.stack([net.w32.double().sum(), net.w32.double().abs().sum()])
        lo, hi = chk.clone(), chk.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        if not bool(torch.equal(lo, hi)):
            raise SystemExit(f"rank {rank}: master weights differ between ranks after the all-reduced update")
        identical = True
    if rank == 0:
        line = dict(metric="resnet50_fwd_bwd_images_per_sec", value=round(value, 1), unit=UNIT, n_gpus=world,
                    steps=args.steps, warmup=args.warmup, ms_per_step=round(ms_per_step, 3), higher_is_better=True,
                    scaling="weak", vs_baseline=None, dtype="bf16", data="synthetic",
                    config=dict(workload="ResNet-50 (bottleneck 3-4-6-3) bf16 fwd+bwd+allreduce+SGD-momentum, NHWC "
                                         "224x224x3(+1 pad), batch 256/GPU, loss scale 1024, 25 MB buckets; not the "
                                         "headline configuration",
                                global_batch=world * batch, parallelism=f"dp{world}",
                                l2="activations (>10 GB per step) far exceed the 126 MB L2; no flush needed",
                                loss=round(float(loss.item()), 4)),
                    clocks=clocks, e2e=e2e, gpu_launches=int(launches // args.steps), roofline=roofline)
        if identical is not None:
            line["weights_identical_on_all_ranks"] = identical
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def cpu_baseline(sample_batch=1, repeats=1):
    """Times the CPU oracle's VGG16-BN step (all host threads) on `sample_batch` images."""
    from oracle import oracle as orc
    from oracle import vgg16bn_cpu as cpu

    orc.lib()
    params = cpu.init_params(seed=1234, image=IMAGE, classes=CLASSES)
    img, labels = cpu.synthetic_batch(100, sample_batch, IMAGE, CLASSES)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        cpu.step(params, img, labels)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return dict(value=round(sample_batch / best, 4), unit=UNIT, cores=orc.num_threads(), kind="port",
                sample=f"one full VGG16-BN step (fwd+bwd+SGD) on {sample_batch} image(s) of 224x224, "
                       f"{best:.1f} s of wall time on {orc.num_threads()} threads")


def run_reference(args):
    """Reference arm: the reference's own CPU implementation of this path cannot be built here (it needs
    mimalloc, Eigen, XNNPACK; its fused block has no CPU launcher at all), so the arm times the oracle's
    loop-for-loop restatement of the reference CPU operators on all host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t_all = time.perf_counter()
    vals = []
    sample = 1
    for i in range(args.warmup + args.steps):
        r = cpu_baseline(sample_batch=sample)
        if i >= args.warmup:
            vals.append(r["value"])
        if time.perf_counter() - t_all > 240:      # stay within a few minutes whatever K and W say
            if not vals:
                vals.append(r["value"])
            break
    value = statistics.mean(vals)
    r["value"] = round(value, 4)
    line = dict(impl="reference", metric=METRIC, value=round(value, 4), unit=UNIT, n_gpus=args.gpus, steps=len(vals),
                warmup=args.warmup, ms_per_step=round(1e3 * sample / value, 1), higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="fp16", data="synthetic",
                config=dict(workload="VGG16-BN AMP fwd+bwd+SGD-momentum, NHWC 224x224x3(+1 pad), CPU restatement of "
                                     "the reference operators, bounded sample of 1 image per step",
                            global_batch=sample, parallelism="cpu"),
                cpu_baseline=r, e2e=dict(value=round(value, 4), unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=BATCH_PER_GPU, help="images per GPU (the metric is quoted at 256)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--bucket-mb", type=float, default=50.0, help="size of a gradient all-reduce bucket")
    ap.add_argument("--bucket-plan", default="tensors", choices=["tensors", "uniform"],
                    help="buckets that end where a weight gradient ends (at least --bucket-mb each), or equal buckets")
    ap.add_argument("--nccl-registered", default="off", choices=["off", "user", "symm"],
                    help="gradient buffer from NCCL's allocator, registered as a user buffer / a symmetric window (N > 1)")
    ap.add_argument("--nccl-high-priority", action="store_true",
                    help="run NCCL's kernels on a high-priority stream (N > 1)")
    ap.add_argument("--workload", default="vgg16bn", choices=["vgg16bn", "resnet50"],
                    help="vgg16bn: the headline configuration; resnet50: BASELINE configuration 4 (information only)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "resnet50":
        run_resnet50(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
