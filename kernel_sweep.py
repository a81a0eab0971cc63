"""Per-kernel roofline sweep of the hot-path kernels on one GPU.

    python kernel_sweep.py                 # everything, JSON lines
    python kernel_sweep.py --only block    # BASELINE.json configuration 2 (one block backward)
    python kernel_sweep.py --only bnrelu --quick
    python kernel_sweep.py --only conv --quick --batch 64 --shape 56,256,256 --what fprop_stats
    python kernel_sweep.py --only fc                   # the classifier layers of VGG16 at batch 256
    python kernel_sweep.py --only resnet50 --cudnn     # ResNet-50 conv shapes, bfloat16

Covers BASELINE.json's config 2 (Conv3x3 C=K=64 + BN + ReLU backward at N=256, 56x56)
and config 5 (BN+ReLU backward over N*H*W x C, fused softmax-CE over N x C), plus the
13 VGG16-BN conv shapes.  Every point: 3 warm-up calls, then timed calls bracketed by
CUDA events on the launching stream with a write over a buffer larger than L2 between
them (not timed); the median is reported.  `frac` = achieved / measured peak
(MEASURED_PEAKS.json beside the repository root when present: copy bandwidth and cuBLAS
bf16 burst rate, these being kernels timed in isolation).

Algorithmic work per call:
    BN+ReLU backward   10.25 B/element  (two sweeps over dy, x, mask; one write of dconv)
    softmax-CE fused   4 B/element + 12 B/row  (read logits, write d_logits)
    conv dgrad / wgrad / fprop   2*N*H*W*K*9*C flop
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import sys

import torch

_ROOT = os.path.dirname(os.path.abspath(__file__))
if _ROOT not in sys.path:
    sys.path.insert(0, _ROOT)

from renaissance_b200 import ops  # noqa: E402


def peaks():
    p = os.path.join(_ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


class Timer:
    def __init__(self, iters):
        self.iters = iters
        self.flush = torch.empty(512 * 1024 * 1024, dtype=torch.uint8, device="cuda")   # 4 x L2

    def __call__(self, fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(self.iters):
            self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return statistics.median(ts), min(ts)


def emit(**kw):
    print(json.dumps(kw), flush=True)


def _library(t, build):
    """Times a cuDNN graph of the reference's path (cudnn_reference.py); {} when not asked for."""
    if not WITH_CUDNN:
        return {}
    try:
        run = build()
        med, _ = t(run)
        return {"cudnn_ms": round(med, 4)}
    except Exception as e:          # an unsupported graph is a result, not a failure of the sweep
        return {"cudnn_ms": None, "cudnn_note": str(e).splitlines()[0][:160]}


def _nhw(m):
    if m == 256 * 56 * 56:
        return (256, 56, 56)
    return (m >> 12, 64, 64) if m % 4096 == 0 else (m, 1, 1)


WITH_CUDNN = False


def bnrelu_point(t, m, c, hbm, src):
    g = torch.Generator(device="cuda").manual_seed(0)
    dy = torch.randn((m, c), generator=g, device="cuda").half()
    x = torch.randn((m, c), generator=g, device="cuda").half()
    bits = torch.randint(0, 256, (m * c // 8,), generator=g, device="cuda", dtype=torch.int32).to(torch.uint8)
    gamma = 1 + 0.2 * torch.randn(c, generator=g, device="cuda")
    mean = x.float().mean(dim=0)
    inv = 1.0 / torch.sqrt(x.float().var(dim=0, unbiased=False) + 1e-5)
    out = torch.empty_like(dy)
    med, best = t(lambda: ops.bnrelu_bwd(dy, bits, x, gamma, mean, inv, dconv=out))
    byt = 10.25 * m * c + 20 * c

    def build():
        import cudnn_reference as cr
        dg, db = torch.empty(c, device="cuda"), torch.empty(c, device="cuda")
        return cr.bnrelu_bwd(dy, bits, x, gamma, mean, inv, torch.empty_like(dy), dg, db, nhw=_nhw(m))

    lib = _library(t, build)
    emit(kernel="bnrelu_bwd (reduce + finalize + apply)", rows=m, channels=c, ms=round(med, 4), best_ms=round(best, 4),
         bound="hbm", achieved=round(byt / med / 1e6, 1), peak=hbm, unit="GB/s", frac=round(byt / med / 1e6 / hbm, 4),
         peak_source=src, **lib)


def softmax_point(t, b, c, ls, hbm, src):
    g = torch.Generator(device="cuda").manual_seed(0)
    z = (torch.randn((b, c), generator=g, device="cuda") * 2).half()
    lab = torch.randint(0, c, (b,), generator=g, device="cuda", dtype=torch.int32)
    sc = torch.tensor([1024.0], device="cuda")
    lsd = torch.tensor([ls], device="cuda")
    d = torch.empty_like(z)
    med, best = t(lambda: ops.softmax_ce_amp_fused(z, lab, sc, lsd, dlogits=d))
    byt = 4.0 * b * c + 12 * b
    emit(kernel="softmax_ce fused fwd+bwd", rows=b, classes=c, label_smoothing=ls, ms=round(med, 4),
         best_ms=round(best, 4), bound="hbm", achieved=round(byt / med / 1e6, 1), peak=hbm, unit="GB/s",
         frac=round(byt / med / 1e6 / hbm, 4), peak_source=src)


def conv_point(t, n, h, c, k, what, tc, src, r=3, pad=1, stride=1, dtype=torch.float16, hbm=None):
    geo = ops.ConvGeometry(n, h, h, c, k, r, r, pad, stride, dtype=dtype)
    oh = geo.oh
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((n, h, h, c), generator=g, device="cuda").to(dtype)
    w = (torch.randn((k, r, r, c), generator=g, device="cuda") * (2.0 / (r * r * c)) ** 0.5).to(dtype)
    dy = torch.randn((n, oh, oh, k), generator=g, device="cuda").to(dtype)
    flop = 2.0 * n * oh * oh * c * k * r * r
    if what == "dgrad":
        dx = torch.empty_like(x)
        med, best = t(lambda: ops.conv_dgrad(geo, dy, w, dx=dx))
    elif what == "wgrad":
        dw = torch.empty_like(w)
        med, best = t(lambda: ops.conv_wgrad(geo, dy, x, dw=dw))
    elif what == "fprop_stats":
        y = torch.empty_like(dy)
        gamma, beta = torch.ones(k, device="cuda"), torch.zeros(k, device="cuda")
        ws = ops.Workspace(torch.device("cuda"))
        med, best = t(lambda: ops.conv_fprop_bn_stats(geo, x, w, gamma, beta, y=y, workspace=ws))
    else:
        y = torch.empty_like(dy)
        med, best = t(lambda: ops.conv_fprop(geo, x, w, y=y))
    ops.device_status()

    def build():
        import cudnn_reference as cr
        if c < 8:
            raise RuntimeError("the reference pads the first layer to 4 channels; cuDNN tensor-core graphs need C % 8 == 0")
        if what == "dgrad":
            return cr.conv_dgrad(dy, w, torch.empty_like(x), pad=pad, stride=stride)
        if what == "wgrad":
            return cr.conv_wgrad(x, dy, torch.empty_like(w), pad=pad, stride=stride)
        if what == "fprop_stats":
            st = (torch.empty(k, device="cuda"), torch.empty(k, device="cuda"))
            return cr.conv_fprop(x, w, torch.empty_like(dy), genstats=st, pad=pad, stride=stride)
        return cr.conv_fprop(x, w, torch.empty_like(dy), pad=pad, stride=stride)

    lib = _library(t, build)
    shape = dict(n=n, h=h, w=h, c=c, k=k)
    extra = {}
    if (r, pad, stride) != (3, 1, 1) or dtype != torch.float16:
        # the ResNet-50 points: 1x1 layers move more bytes per flop than the tensor pipe can hide, so the
        # HBM figure (activations in and out once, filters once) is reported beside the flop rate
        shape.update(r=r, pad=pad, stride=stride)
        byt = 2.0 * (n * oh * oh * k + n * h * h * c + k * r * r * c)
        extra = dict(dtype=str(dtype).replace("torch.", ""), tensor_cores=ops.conv_uses_tensor_cores(
            geo, "fprop" if what.startswith("fprop") else what), hbm_gbs=round(byt / med / 1e6, 1))
        if hbm:
            extra["hbm_frac"] = round(byt / med / 1e6 / hbm, 4)
    emit(kernel=f"conv {what}", shape=shape, ms=round(med, 4), best_ms=round(best, 4),
         bound="tensor", achieved=round(flop / med / 1e9, 1), peak=tc, unit="TFLOP/s",
         frac=round(flop / med / 1e9 / tc, 4), peak_source=src, **extra, **lib)


def block_point(t, n, h, c, k, hbm, tc, src):
    """BASELINE.json configuration 2: the whole block backward through trb200_cbr_bwd on three streams."""
    geo = ops.ConvGeometry(n, h, h, c, k)
    g = torch.Generator(device="cuda").manual_seed(1)
    x0 = torch.randn((n, h, h, c), generator=g, device="cuda").half()
    x = x0.clone()
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
    torch.cuda.synchronize()

    def call():
        with torch.cuda.stream(st.bn):
            ops.cbr_amp_bwd(geo, dy, w, gamma, mean, inv, bits, x, conv_out, bn_scratch=scratch, dw=dw, streams=st)
        torch.cuda.current_stream().wait_stream(st.bn)

    torch.cuda.current_stream().wait_stream(st.bn)
    med, best = t(call)
    ops.device_status()
    flop = 2 * 2.0 * n * h * h * c * k * 9
    byt = 10.25 * n * h * h * k
    emit(kernel="cbr_amp_bwd (BN+ReLU bwd, wgrad, dgrad)", shape=dict(n=n, h=h, w=h, c=c, k=k), ms=round(med, 4),
         best_ms=round(best, 4), ideal_ms=round(flop / tc / 1e9 + byt / hbm / 1e6, 4),
         note="ideal = conv flop at the measured tensor peak + BN bytes at the measured copy bandwidth",
         frac=round((flop / tc / 1e9 + byt / hbm / 1e6) / med, 4), peak_source=src)


# ResNet-50's distinct convolutions: kernel, in channels, out channels, input extent, stride, padding
RESNET50_CONVS = [
    (7, 4, 64, 224, 2, 3),
    (1, 64, 64, 56, 1, 0), (3, 64, 64, 56, 1, 1), (1, 64, 256, 56, 1, 0), (1, 256, 64, 56, 1, 0),
    (1, 256, 128, 56, 1, 0), (1, 256, 512, 56, 2, 0), (3, 128, 128, 56, 2, 1),
    (1, 128, 512, 28, 1, 0), (1, 512, 128, 28, 1, 0), (3, 128, 128, 28, 1, 1),
    (1, 512, 256, 28, 1, 0), (1, 512, 1024, 28, 2, 0), (3, 256, 256, 28, 2, 1),
    (1, 256, 1024, 14, 1, 0), (1, 1024, 256, 14, 1, 0), (3, 256, 256, 14, 1, 1),
    (1, 1024, 512, 14, 1, 0), (1, 1024, 2048, 14, 2, 0), (3, 512, 512, 14, 2, 1),
    (1, 512, 2048, 7, 1, 0), (1, 2048, 512, 7, 1, 0), (3, 512, 512, 7, 1, 1),
]

VGG_SHAPES = [(224, 64, 64), (112, 64, 128), (112, 128, 128), (56, 128, 256), (56, 256, 256), (28, 256, 512),
              (28, 512, 512), (14, 512, 512)]



def softmax_split_point(t, b, c, hbm, src):
    """The two separate nodes as the registry adapter runs them when the graph is not patched for the fused kernel:
    SOFTMAX_CE_AMP_FWD (logits -> float probabilities + loss) and SOFTMAX_CE_AMP_BWD (probabilities -> half d_logits):
    2 + 4 bytes written and read per class in the forward, 4 + 2 in the backward = 12 B per class."""
    g = torch.Generator(device="cuda").manual_seed(0)
    z = (torch.randn((b, c), generator=g, device="cuda") * 2).half()
    lab = torch.randint(0, c, (b,), generator=g, device="cuda", dtype=torch.int32)
    sc = torch.tensor([1024.0], device="cuda")
    lsd = torch.tensor([0.0], device="cuda")
    probs = torch.empty((b, c), dtype=torch.float32, device="cuda")
    d = torch.empty_like(z)
    fwd = ops.softmax_ce_amp_fwd(z, lab, lsd, probs=probs)

    def both():
        f = ops.softmax_ce_amp_fwd(z, lab, lsd, probs=probs)
        ops.softmax_ce_amp_bwd(probs, lab, sc, f["inv_scaling"], lsd, dlogits=d)

    med, best = t(both)
    byt = 12.0 * b * c + 12 * b
    emit(kernel="softmax_ce split nodes (fwd with probs, bwd)", rows=b, classes=c, label_smoothing=0.0, ms=round(med, 4),
         best_ms=round(best, 4), bound="hbm", achieved=round(byt / med / 1e6, 1), peak=hbm, unit="GB/s",
         frac=round(byt / med / 1e6 / hbm, 4), peak_source=src)


def pool_point(t, n, h, c, hbm, src):
    """The block's HBM-bound kernels around a 2x2 max pool: BN apply + ReLU + mask + pool forward, and the pool + BN +
    ReLU backward (bytes per full-resolution element: 2.875 and 7.75), and the forward without a pool (4.125)."""
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((n, h, h, c), generator=g, device="cuda").half()
    sc = 0.5 + torch.rand(c, generator=g, device="cuda")
    bi = 0.3 * torch.randn(c, generator=g, device="cuda")
    po, am, mb = ops.bn_apply_relu_mask_pool(x, sc, bi)
    e = x.numel()
    med, best = t(lambda: ops.bn_apply_relu_mask_pool(x, sc, bi, mask_bits=mb, pool_out=po, argmax=am))
    emit(kernel="bn_apply_relu_mask_pool (forward)", shape=dict(n=n, h=h, w=h, c=c), ms=round(med, 4), best_ms=round(best, 4),
         bound="hbm", achieved=round(2.875 * e / med / 1e6, 1), peak=hbm, unit="GB/s",
         frac=round(2.875 * e / med / 1e6 / hbm, 4), peak_source=src)
    dy = torch.randn((n, h // 2, h // 2, c), generator=g, device="cuda").half()
    gamma = 1 + 0.2 * torch.randn(c, generator=g, device="cuda")
    mean = 0.1 * torch.randn(c, generator=g, device="cuda")
    inv = 0.5 + torch.rand(c, generator=g, device="cuda")
    out = torch.empty_like(x)
    med, best = t(lambda: ops.bnrelu_pool_bwd(dy, am, mb, x, gamma, mean, inv, dconv=out))
    emit(kernel="bnrelu_pool_bwd (reduce + finalize + apply)", shape=dict(n=n, h=h, w=h, c=c), ms=round(med, 4),
         best_ms=round(best, 4), bound="hbm", achieved=round(7.75 * e / med / 1e6, 1), peak=hbm, unit="GB/s",
         frac=round(7.75 * e / med / 1e6 / hbm, 4), peak_source=src)
    y = out
    med, best = t(lambda: ops.bn_apply_relu_mask(x, sc, bi, relu_out=y, mask_bits=mb))
    emit(kernel="bn_apply_relu_mask (forward)", shape=dict(n=n, h=h, w=h, c=c), ms=round(med, 4), best_ms=round(best, 4),
         bound="hbm", achieved=round(4.125 * e / med / 1e6, 1), peak=hbm, unit="GB/s",
         frac=round(4.125 * e / med / 1e6 / hbm, 4), peak_source=src)

def fc_point(t, batch, in_f, out_f, hbm, src):
    """A classifier layer at batch 256: forward (y = x.w^T + b with ReLU) and backward (dx, float dW as the
    reference's FC_AMP_BWD writes it, db).  Both are bound by the weight matrix in HBM: the forward reads it once
    (2 B per weight), the backward reads it once and writes the float gradient (6 B per weight)."""
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((batch, in_f), generator=g, device="cuda").half()
    w = (torch.randn((out_f, in_f), generator=g, device="cuda") * (2.0 / in_f) ** 0.5).half()
    b = torch.zeros(out_f, device="cuda")
    dy = torch.randn((batch, out_f), generator=g, device="cuda").half()
    y = ops.fc_amp_fwd(x, w, b, relu=True)
    dx = torch.empty_like(x)
    dw = torch.empty((out_f, in_f), dtype=torch.float32, device="cuda")
    db = torch.empty(out_f, device="cuda")
    wb = float(in_f) * out_f
    act = 2.0 * batch * (in_f + out_f)
    med, best = t(lambda: ops.fc_amp_fwd(x, w, b, relu=True, y=y))
    byt = 2 * wb + act
    emit(kernel="fc_amp_fwd (gemm_skinny_kernel + fc_bias_act_kernel)", shape=dict(batch=batch, in_features=in_f, out_features=out_f),
         ms=round(med, 4), best_ms=round(best, 4), bound="hbm", achieved=round(byt / med / 1e6, 1), peak=hbm, unit="GB/s",
         frac=round(byt / med / 1e6 / hbm, 4), peak_source=src)
    med, best = t(lambda: ops.fc_amp_bwd(dy, w, x, dx=dx, dw=dw, db=db))
    byt = 6 * wb + 2 * act
    emit(kernel="fc_amp_bwd (dW float, dx, db)", shape=dict(batch=batch, in_features=in_f, out_features=out_f),
         ms=round(med, 4), best_ms=round(best, 4), bound="hbm", achieved=round(byt / med / 1e6, 1), peak=hbm, unit="GB/s",
         frac=round(byt / med / 1e6 / hbm, 4), peak_source=src)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="all", choices=["all", "block", "bnrelu", "pool", "softmax", "conv", "fc", "resnet50"])
    ap.add_argument("--quick", action="store_true", help="one small point per kernel (for profiler captures)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--batch", type=int, default=256, help="images for the conv / block points")
    ap.add_argument("--cudnn", action="store_true",
                    help="also time the reference's cuDNN-frontend graphs for the conv and BN+ReLU points (cudnn_ms)")
    ap.add_argument("--shape", default="", help="H,C,K: only this conv shape (with --only conv); ROWS,CLASSES with --only softmax")
    ap.add_argument("--what", default="", help="comma list out of dgrad,wgrad,fprop,fprop_stats (with --only conv)")
    args = ap.parse_args()
    global WITH_CUDNN
    WITH_CUDNN = args.cudnn
    hbm, tc, src = peaks()
    t = Timer(1 if args.quick else args.iters)
    n = args.batch
    if args.only in ("all", "block"):
        block_point(t, n, 56, 64, 64, hbm, tc, src)
    if args.only in ("all", "bnrelu"):
        pts = [(n * 56 * 56, 64)] if args.quick else \
            [(1 << e, c) for c in (64, 256, 512, 2048) for e in (16, 18, 20, 22, 24) if (1 << e) * c * 2 * 3 < 150e9]
        if not args.quick:
            pts.insert(0, (256 * 56 * 56, 64))
        for m, c in pts:
            bnrelu_point(t, m, c, hbm, src)
    if args.only in ("all", "pool"):
        # the pooled layers of VGG16-BN; --shape H,C picks one, --batch the images
        pts = [(224, 64)] if args.quick else [(224, 64), (112, 128), (56, 256), (28, 512), (14, 512)]
        if args.shape and args.only == "pool":
            pts = [tuple(int(v) for v in args.shape.split(","))[:2]]
        for h, c in pts:
            pool_point(t, n, h, c, hbm, src)
    if args.only in ("all", "softmax"):
        pts = [(4096, 32000, 0.1)] if args.quick else \
            [(b, c, ls) for b in (4096, 65536) for c in (1000, 10000, 32000) for ls in (0.0, 0.1)] + [(256, 1000, 0.0)]
        if args.shape and args.only == "softmax":
            b, c = (int(v) for v in args.shape.split(","))
            pts = [(b, c, 0.0)]
        for b, c, ls in pts:
            softmax_point(t, b, c, ls, hbm, src)
        if not args.quick and not args.shape:
            for b, c in ((65536, 1000), (65536, 10000), (16384, 32000)):
                softmax_split_point(t, b, c, hbm, src)
    if args.only in ("all", "conv"):
        shapes = [(56, 64, 64), (28, 256, 512)] if args.quick else [(56, 64, 64)] + VGG_SHAPES
        if args.shape and args.only == "conv":
            shapes = [tuple(int(v) for v in args.shape.split(","))]
        kinds = tuple(args.what.split(",")) if args.what else ("dgrad", "wgrad", "fprop", "fprop_stats")
        for h, c, k in shapes:
            for what in kinds:
                conv_point(t, n, h, c, k, what, tc, src)
    if args.only in ("all", "fc"):
        for in_f, out_f in ([(25088, 4096)] if args.quick else [(25088, 4096), (4096, 4096), (4096, 1024)]):
            fc_point(t, 256, in_f, out_f, hbm, src)
    if args.only == "resnet50":
        # BASELINE.json configuration 4 at the level the hot path reaches it: the data and weight gradients of every
        # distinct convolution of ResNet-50 on bfloat16 tensors
        kinds = tuple(args.what.split(",")) if args.what else ("dgrad", "wgrad")
        for r, c, k, h, stride, pad in RESNET50_CONVS:
            for what in kinds:
                if what.startswith("fprop") and not ops.conv_uses_tensor_cores(
                        ops.ConvGeometry(n, h, h, c, k, r, r, pad, stride, dtype=torch.bfloat16), "fprop"):
                    continue
                conv_point(t, n, h, c, k, what, tc, src, r=r, pad=pad, stride=stride, dtype=torch.bfloat16, hbm=hbm)


if __name__ == "__main__":
    main()
