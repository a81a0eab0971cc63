#!/usr/bin/env python3
"""Regenerate the golden vectors under tests/golden/.

The reference project stores no expected numbers: each of its operator tests
asks PyTorch for them at run time (tests/op/test_conv_fwd_bwd.py,
tests/op/test_bn_fwd_bwd_legacy.py, tests/correction/test_softmax_ce.py,
tests/correction/test_mlp_final.py).  This script follows the same recipes --
PyTorch CPU ops / autograd in fp32 on NCHW views of NHWC data -- on small
shapes, and writes inputs and expected outputs to ``.npz`` files.  Inputs come
from ``numpy.random.default_rng`` so that they do not depend on the torch
version.  Nothing here imports the oracle or the CUDA library.

    python tests/golden/make_golden.py
"""
import os

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
torch.set_num_threads(1)
torch.use_deterministic_algorithms(True)


def save(name, **arrays):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **arrays)
    print(f"{name}.npz  {os.path.getsize(path) / 1024:.1f} KiB")


def nchw(a):
    return torch.from_numpy(np.ascontiguousarray(a)).permute(0, 3, 1, 2).contiguous()


def nhwc(t):
    return t.permute(0, 2, 3, 1).contiguous().numpy()


def conv_case(name, seed, n, h, w, c, k, ker, stride, pad, half):
    """Recipe of tests/op/test_conv_fwd_bwd.py: conv2d, conv_transpose2d for dX,
    autograd for dW, per-channel sum / sum of squares of Y."""
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal((n, h, w, c)) * 0.5).astype(np.float32)
    wt = (rng.standard_normal((k, ker, ker, c)) * 0.1).astype(np.float32)
    oh = (h + 2 * pad - ker) // stride + 1
    ow = (w + 2 * pad - ker) // stride + 1
    dy = (rng.standard_normal((n, oh, ow, k)) * 0.5).astype(np.float32)
    if half:
        x, wt, dy = (a.astype(np.float16).astype(np.float32) for a in (x, wt, dy))
    xt = nchw(x).requires_grad_(True)
    wtt = nchw(wt).requires_grad_(True)
    y = F.conv2d(xt, wtt, stride=stride, padding=pad)
    y.backward(nchw(dy))
    dx_t = F.conv_transpose2d(nchw(dy), wtt.detach(), stride=stride, padding=pad)
    # the reference's generator takes dX from conv_transpose2d; autograd is the same
    # thing whenever the stride tiles the input, and stays right when it does not
    if dx_t.shape[2] >= h and dx_t.shape[3] >= w:
        assert torch.allclose(dx_t[:, :, :h, :w], xt.grad, atol=1e-5)
    yd = y.detach()
    save(name, x=x, w=wt, dy=dy, y=nhwc(yd), dx=nhwc(xt.grad), dw=nhwc(wtt.grad),
         ysum=yd.sum(dim=(0, 2, 3)).numpy(), ysqsum=(yd ** 2).sum(dim=(0, 2, 3)).numpy(),
         params=np.array([n, h, w, c, k, ker, stride, pad, int(half)], np.int32))


def bn_case(name, seed, n, h, w, c, eps=1e-5, momentum=0.1):
    """Recipe of tests/op/test_bn_fwd_bwd_legacy.py: biased variance for inv_std,
    unbiased for the running variance, autograd through the batch statistics."""
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal((n, h, w, c)) * 0.5).astype(np.float32)
    gamma = (1.0 + rng.standard_normal(c) * 0.2).astype(np.float32)
    beta = (rng.standard_normal(c) * 0.2).astype(np.float32)
    dy = (rng.standard_normal((n, h, w, c)) * 0.5).astype(np.float32)
    xt = nchw(x).requires_grad_(True)
    g = torch.from_numpy(gamma).requires_grad_(True)
    b = torch.from_numpy(beta).requires_grad_(True)
    mean = xt.mean(dim=(0, 2, 3))
    var = xt.var(dim=(0, 2, 3), unbiased=False)
    inv_std = 1.0 / torch.sqrt(var + eps)
    y = (xt - mean.view(1, c, 1, 1)) * inv_std.view(1, c, 1, 1) * g.view(1, c, 1, 1) + b.view(1, c, 1, 1)
    y.backward(nchw(dy))
    rm = (1 - momentum) * torch.zeros(c) + momentum * mean.detach()
    rv = (1 - momentum) * torch.ones(c) + momentum * xt.detach().var(dim=(0, 2, 3), unbiased=True)
    save(name, x=x, gamma=gamma, beta=beta, dy=dy, y=nhwc(y.detach()),
         saved_mean=mean.detach().numpy(), saved_inv_std=inv_std.detach().numpy(),
         running_mean=rm.numpy(), running_var=rv.numpy(),
         dx=nhwc(xt.grad), dgamma=g.grad.numpy(), dbeta=b.grad.numpy(),
         params=np.array([n, h, w, c], np.int32), eps=np.float32(eps), momentum=np.float32(momentum))


def softmax_case(name, seed, batch, classes, half, ls=0.0, scaling=1.0):
    """Recipe of tests/correction/test_softmax_ce.py: log_softmax in fp32, mean CE,
    d_logits = (softmax - onehot) * scaling / batch.  With label smoothing (not
    covered by the reference's generator) the expected values come from
    F.cross_entropy(label_smoothing=ls) and autograd."""
    rng = np.random.default_rng(seed)
    z = (rng.standard_normal((batch, classes)) * 0.5).astype(np.float32)
    if half:
        z = z.astype(np.float16).astype(np.float32)
    labels = rng.integers(0, classes, size=batch).astype(np.int32)
    zt = torch.from_numpy(z).requires_grad_(True)
    lt = torch.from_numpy(labels).long()
    loss = F.cross_entropy(zt, lt, label_smoothing=ls)
    (loss * scaling).backward()
    probs = F.softmax(zt.detach(), dim=1)
    pred = probs.argmax(dim=1).to(torch.int32)
    save(name, logits=z, labels=labels, loss=np.float32(loss.item()), probs=probs.numpy(),
         dlogits=zt.grad.numpy(), pred=pred.numpy(),
         params=np.array([batch, classes, int(half)], np.int32), ls=np.float32(ls),
         scaling=np.float32(scaling))


def cbr_case(name, seed, n, h, w, c, k, first_layer=False):
    """Conv3x3(s1,p1) + BatchNorm(training) + ReLU on half inputs, the composition
    tests/op/test_cbr_amp_bwd.cpp compares the fused op with; forward and backward
    by autograd in fp32 (intermediates are NOT rounded to half here, so parity with
    the half-rounded path is to fp16 tolerance)."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, h, w, c)).astype(np.float16)
    wt = (rng.standard_normal((k, 3, 3, c)) * np.sqrt(2.0 / (9 * c))).astype(np.float16)
    gamma = (1.0 + rng.standard_normal(k) * 0.2).astype(np.float32)
    beta = (rng.standard_normal(k) * 0.2).astype(np.float32)
    dy = rng.standard_normal((n, h, w, k)).astype(np.float16)
    xt = nchw(x.astype(np.float32)).requires_grad_(True)
    wtt = nchw(wt.astype(np.float32)).requires_grad_(True)
    g = torch.from_numpy(gamma).requires_grad_(True)
    b = torch.from_numpy(beta).requires_grad_(True)
    conv = F.conv2d(xt, wtt, padding=1)
    y = F.batch_norm(conv, None, None, g, b, training=True, eps=1e-5)
    out = F.relu(y)
    out.backward(nchw(dy.astype(np.float32)))
    mean = conv.detach().mean(dim=(0, 2, 3))
    var = conv.detach().var(dim=(0, 2, 3), unbiased=False)
    save(name, x=x, w=wt, gamma=gamma, beta=beta, dy=dy,
         conv_out=nhwc(conv.detach()), relu_out=nhwc(out.detach()),
         mask=(nhwc(y.detach()) > 0).astype(np.int8),
         saved_mean=mean.numpy(), saved_inv_std=(1.0 / torch.sqrt(var + 1e-5)).numpy(),
         dx=nhwc(xt.grad), dw=nhwc(wtt.grad), dgamma=g.grad.numpy(), dbeta=b.grad.numpy(),
         params=np.array([n, h, w, c, k, int(first_layer)], np.int32))


def mlp_case(name, seed, sizes, batch, lr, full=True):
    """BASELINE.json configuration 1: Linear+ReLU MLP, softmax-CE (mean), one SGD step.  With
    full=False only scalars and a few slices are stored (the tensors are rebuilt
    from the seed by the test)."""
    rng = np.random.default_rng(seed)
    x = rng.random((batch, sizes[0]), dtype=np.float32)
    labels = rng.integers(0, sizes[-1], size=batch).astype(np.int32)
    ws = [(rng.standard_normal((o, i)) * np.sqrt(2.0 / i)).astype(np.float32)
          for i, o in zip(sizes[:-1], sizes[1:])]
    bs = [np.zeros(o, np.float32) for o in sizes[1:]]
    wt = [torch.from_numpy(a.copy()).requires_grad_(True) for a in ws]
    bt = [torch.from_numpy(a.copy()).requires_grad_(True) for a in bs]
    hcur = torch.from_numpy(x)
    for li, (w_, b_) in enumerate(zip(wt, bt)):
        hcur = F.linear(hcur, w_, b_)
        if li + 1 < len(wt):
            hcur = F.relu(hcur)
    loss = F.cross_entropy(hcur, torch.from_numpy(labels).long())
    loss.backward()
    out = dict(sizes=np.array(sizes, np.int32), batch=np.int32(batch), lr=np.float32(lr),
               seed=np.int32(seed), loss=np.float32(loss.item()), logits=hcur.detach().numpy())
    for li, (w_, b_) in enumerate(zip(wt, bt)):
        w_new = (w_.detach() - lr * w_.grad).numpy()
        b_new = (b_.detach() - lr * b_.grad).numpy()
        if full:
            out[f"w{li}_new"], out[f"b{li}_new"] = w_new, b_new
            out[f"dw{li}"], out[f"db{li}"] = w_.grad.numpy(), b_.grad.numpy()
        else:
            out[f"w{li}_new_head"] = w_new[:4, :16].copy()
            out[f"b{li}_new"] = b_new
            out[f"dw{li}_norm"] = np.float32(w_.grad.norm().item())
    if full:
        out.update(x=x, labels=labels, **{f"w{li}": a for li, a in enumerate(ws)})
    save(name, **out)


if __name__ == "__main__":
    conv_case("conv_fp32_3x3_s1", 11, 2, 8, 8, 8, 16, 3, 1, 1, False)
    conv_case("conv_fp32_3x3_s2", 12, 2, 9, 7, 4, 8, 3, 2, 1, False)
    conv_case("conv_fp32_7x7_s2", 13, 1, 12, 12, 3, 8, 7, 2, 3, False)
    conv_case("conv_fp16_3x3_s1", 14, 2, 8, 8, 16, 16, 3, 1, 1, True)
    bn_case("bn2d_fp32", 21, 4, 5, 5, 8)
    bn_case("bn1d_fp32", 22, 16, 1, 1, 10)
    softmax_case("softmax_fp32_1000", 31, 8, 1000, False)
    softmax_case("softmax_fp16_1000", 32, 8, 1000, True)
    softmax_case("softmax_fp32_10", 33, 16, 10, False)
    softmax_case("softmax_fp16_ls", 34, 8, 100, True, ls=0.1, scaling=1024.0)
    cbr_case("cbr_block_small", 41, 4, 8, 8, 16, 32)
    cbr_case("cbr_block_first", 42, 2, 8, 8, 4, 16, first_layer=True)
    mlp_case("mlp_small", 51, [32, 16, 12, 10], 8, 0.1, full=True)
    mlp_case("mlp_config1", 52, [784, 512, 256, 10], 128, 0.1, full=False)
