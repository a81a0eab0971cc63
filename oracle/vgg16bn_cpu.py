"""One VGG16-BN AMP training step on the CPU oracle.

TEST INFRASTRUCTURE ONLY (checker for the GPU step driver and the timed CPU
baseline).  The step is composed from the oracle's restatements of the reference
operators, in the order of the reference's training loop
(src/task/deep_learning_task.cpp:1162-1217):

    13 x CBR_AMP_FWD  (conv, batch statistics, BN apply + ReLU + mask)   cbr_op.cpp:430-718
    5  x max pool 2x2                                                     maxpool_op.cu:23-217
    FC + ReLU (+ dropout mask given by the caller), FC + ReLU, FC         fc_op.cpp:802-898
    softmax-CE forward / backward with the loss scale                     softmax_ce_op.cu:63-177, 438-468
    FC backward, 13 x CBR_AMP_BWD (the first without dgrad)              cbr_op.cpp:1359-1651
    SGD with momentum on float master weights, half working copy          optimizer_op.cpp:306-313

Half tensors are rounded where the GPU path stores half (activations, weight
gradients, the FC activations), so a step here and a step of the GPU driver agree
to half precision.
"""
from __future__ import annotations

import math
import time

import numpy as np

from . import oracle as orc

CFG = [64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M"]


def h16(a):
    return np.asarray(a, np.float32).astype(np.float16)


def init_params(seed=0, image=224, classes=1000, fc_width=4096):
    """Kaiming-normal float master weights; conv weights KRSC with the input padded 3 -> 4."""
    rng = np.random.default_rng(seed)
    convs, c, h = [], 4, image
    for v in CFG:
        if v == "M":
            h //= 2
            continue
        fan_in = 9 * (3 if not convs else c)
        w = (rng.standard_normal((v, 3, 3, c)) * math.sqrt(2.0 / fan_in)).astype(np.float32)
        if not convs:
            w[..., 3] = 0.0
        convs.append(dict(w=w, gamma=np.ones(v, np.float32), beta=np.zeros(v, np.float32)))
        c = v
    dims = [(h * h * c, fc_width), (fc_width, fc_width), (fc_width, classes)]
    fcs = [dict(w=(rng.standard_normal((o, i)) * math.sqrt(2.0 / i)).astype(np.float32), b=np.zeros(o, np.float32))
           for i, o in dims]
    return dict(convs=convs, fcs=fcs)


def step(params, images16, labels, lr=0.01, momentum=0.9, weight_decay=5e-4, loss_scale=1024.0,
         label_smoothing=0.0, dropout_keep=None, momentum_buf=None, timings=None, stats_from_half=True):
    """Forward + backward + optimizer.  `params` is updated in place (float master weights).
    dropout_keep: optional list of two float arrays (already scaled by 1/(1-p)) or None.
    stats_from_half: batch statistics from the stored half conv output (what the GPU driver does today)
    rather than from the float accumulator (what cuDNN's genstats epilogue does).
    Returns dict(loss, grads) where grads mirror `params` (float, still multiplied by the loss scale)."""
    t0 = time.perf_counter()
    n = images16.shape[0]
    x = images16
    saved = []
    pool_after = [i + 1 < len(CFG) and CFG[i + 1] == "M" for i, v in enumerate(CFG) if v != "M"]
    for L, pool in zip(params["convs"], pool_after):
        f = orc.cbr_fwd_amp(x, h16(L["w"]), L["gamma"], L["beta"], stats_from_half=stats_from_half)
        rec = dict(x=x, fwd=f)
        y = f["relu_out"]
        if pool:
            y, am = orc.maxpool2x2_fwd(y)
            rec["argmax"] = am
        saved.append(rec)
        x = y
    a = x.reshape(n, -1)
    fc_in, z = [a], None
    for j, f in enumerate(params["fcs"]):
        z = h16(orc.fc_fwd(a.astype(np.float32), h16(f["w"]).astype(np.float32), h16(f["b"]).astype(np.float32)))
        if j < 2:
            z = np.maximum(z, np.float16(0))
            if dropout_keep is not None:
                z = h16(z.astype(np.float32) * dropout_keep[j])
            fc_in.append(z)
            a = z
    sm = orc.softmax_ce_amp(z, labels, scaling=loss_scale, ls=label_smoothing, want_probs=False)
    t1 = time.perf_counter()

    grads = dict(convs=[None] * len(params["convs"]), fcs=[None] * 3)
    dz = sm["dlogits"]
    for j in reversed(range(3)):
        f = params["fcs"][j]
        dx, dw, db = orc.fc_bwd(dz.astype(np.float32), h16(f["w"]).astype(np.float32), fc_in[j].astype(np.float32))
        grads["fcs"][j] = dict(w=h16(dw).astype(np.float32), b=h16(db).astype(np.float32))
        dx = h16(dx)
        if j > 0:
            if dropout_keep is not None:
                dx = h16(dx.astype(np.float32) * dropout_keep[j - 1])
            dx = np.where(fc_in[j] > 0, dx, np.float16(0))
        dz = dx
    last = saved[-1]["fwd"]["relu_out"]
    g = dz.reshape(n, last.shape[1] // 2, last.shape[2] // 2, last.shape[3]) if "argmax" in saved[-1] else dz.reshape(last.shape)
    for i in reversed(range(len(saved))):
        rec, L = saved[i], params["convs"][i]
        f = rec["fwd"]
        if "argmax" in rec:
            g = orc.maxpool2x2_bwd(g, rec["argmax"], f["relu_out"].shape)
        out = orc.cbr_bwd_amp(g, h16(L["w"]), L["gamma"], f["saved_mean"], f["saved_inv_std"], f["mask_bits"],
                              rec["x"], f["conv_out"], first_layer=(i == 0))
        grads["convs"][i] = dict(w=out["dw"].astype(np.float32), gamma=out["dgamma"], beta=out["dbeta"])
        g = out["dx"]
    t2 = time.perf_counter()

    if momentum_buf is None:
        momentum_buf = dict(convs=[{k: np.zeros_like(v) for k, v in L.items()} for L in params["convs"]],
                            fcs=[{k: np.zeros_like(v) for k, v in f.items()} for f in params["fcs"]])
    for group in ("convs", "fcs"):
        for p, gr, mb in zip(params[group], grads[group], momentum_buf[group]):
            for key in p:
                p[key], mb[key] = orc.momentum(p[key].ravel(), gr[key].ravel(), mb[key].ravel(), lr, weight_decay,
                                               momentum, loss_scale)
                p[key] = p[key].reshape(gr[key].shape)
                mb[key] = mb[key].reshape(gr[key].shape)
    t3 = time.perf_counter()
    if timings is not None:
        timings.update(forward_s=t1 - t0, backward_s=t2 - t1, optimizer_s=t3 - t2)
    return dict(loss=sm["loss"], grads=grads, logits=z, momentum=momentum_buf)


def synthetic_batch(seed, batch, image=224, classes=1000):
    """images ~ N(0,1) as half NHWC with the 4th channel zero, labels uniform."""
    rng = np.random.default_rng(seed)
    img = np.zeros((batch, image, image, 4), np.float16)
    img[..., :3] = rng.standard_normal((batch, image, image, 3)).astype(np.float16)
    labels = rng.integers(0, classes, size=batch).astype(np.int32)
    return img, labels
