"""One whole VGG16-BN training step of the GPU driver against the CPU oracle's step
(small images so that the oracle finishes in seconds), and the forward-side kernels."""
import numpy as np
import pytest
import torch

from conftest import rel_l2, rel_max
from gpu_util import dev, host

pytestmark = pytest.mark.gpu


def test_bn_apply_relu_mask_is_bit_exact(orc):
    """ReLU masks must be bit-exact: same eq_scale / eq_bias in, same bits out."""
    from renaissance_b200 import ops
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2, 9, 7, 16)).astype(np.float16)
    w = (rng.standard_normal((24, 3, 3, 16)) * 0.1).astype(np.float16)
    gamma = (1 + 0.3 * rng.standard_normal(24)).astype(np.float32)
    beta = (0.3 * rng.standard_normal(24)).astype(np.float32)
    f = orc.cbr_fwd_amp(x, w, gamma, beta, round_steps=True)
    y, bits = ops.bn_apply_relu_mask(dev(f["conv_out"]), dev(f["eq_scale"]), dev(f["eq_bias"]))
    torch.cuda.synchronize()
    assert np.array_equal(host(bits), f["mask_bits"])
    assert np.array_equal(host(y).view(np.uint16), f["relu_out"].view(np.uint16))


def test_bn_stats_finalize_matches_oracle(orc):
    from renaissance_b200 import ops
    rng = np.random.default_rng(4)
    m, c = 5000, 64
    co = (rng.standard_normal((m, c)) * 1.3 + 0.4).astype(np.float16)
    gamma = (1 + 0.2 * rng.standard_normal(c)).astype(np.float32)
    beta = (0.2 * rng.standard_normal(c)).astype(np.float32)
    rm, rv = torch.zeros(c, device="cuda"), torch.ones(c, device="cuda")
    out = ops.bn_stats_finalize(dev(co), dev(gamma), dev(beta), running_mean=rm, running_var=rv, want_sums=True)
    torch.cuda.synchronize()
    rm_ref, rv_ref = np.zeros(c, np.float32), np.ones(c, np.float32)
    _, mean, inv = orc.bn_fwd(co.astype(np.float32), gamma, beta, rm_ref, rv_ref)
    assert rel_max(host(out["sum"]), co.astype(np.float64).sum(axis=0)) < 1e-4
    assert rel_max(host(out["sqsum"]), (co.astype(np.float64) ** 2).sum(axis=0)) < 1e-4
    assert np.abs(host(out["saved_mean"]) - mean).max() < 1e-5
    assert rel_max(host(out["saved_inv_std"]), inv) < 1e-4
    assert rel_max(host(out["eq_scale"]), gamma * inv) < 1e-4
    assert np.abs(host(out["eq_bias"]) - (beta - mean * gamma * inv)).max() < 1e-4
    assert np.abs(host(rm) - rm_ref).max() < 1e-5 and rel_max(host(rv), rv_ref) < 1e-4


@pytest.mark.parametrize("n,h,w,c,k", [(2, 8, 8, 64, 64), (3, 7, 5, 64, 128), (2, 14, 14, 128, 512), (2, 12, 10, 4, 64),
                                       (5, 9, 9, 256, 256)])
def test_conv_with_statistics_in_its_epilogue(orc, n, h, w, c, k):
    """conv + batch statistics + bn_finalize in two launches: the conv output must equal the plain
    conv kernel's bit for bit, the statistics must be those of that (half) output."""
    from renaissance_b200 import ops
    rng = np.random.default_rng(n + h + k)
    x = rng.standard_normal((n, h, w, c)).astype(np.float16)
    wt = (rng.standard_normal((k, 3, 3, c)) * np.sqrt(2.0 / (9 * c))).astype(np.float16)
    gamma = (1 + 0.2 * rng.standard_normal(k)).astype(np.float32)
    beta = (0.2 * rng.standard_normal(k)).astype(np.float32)
    geo = ops.ConvGeometry(n, h, w, c, k)
    y_plain = ops.conv_fprop(geo, dev(x), dev(wt))
    rm, rv = torch.zeros(k, device="cuda"), torch.ones(k, device="cuda")
    y, st = ops.conv_fprop_bn_stats(geo, dev(x), dev(wt), dev(gamma), dev(beta), running_mean=rm, running_var=rv,
                                    want_sums=True)
    ops.device_status()
    assert torch.equal(y, y_plain)
    yf = host(y).astype(np.float64).reshape(-1, k)
    m = yf.shape[0]
    assert rel_max(host(st["sum"]), yf.sum(axis=0)) < 1e-4
    assert rel_max(host(st["sqsum"]), (yf ** 2).sum(axis=0)) < 1e-4
    mean = yf.mean(axis=0)
    inv = 1.0 / np.sqrt(yf.var(axis=0) + 1e-5)
    assert np.abs(host(st["saved_mean"]) - mean).max() < 1e-5
    assert rel_max(host(st["saved_inv_std"]), inv) < 1e-4
    assert rel_max(host(st["eq_scale"]), gamma * inv) < 1e-4
    assert np.abs(host(st["eq_bias"]) - (beta - mean * gamma * inv)).max() < 1e-4
    assert np.abs(host(rm) - 0.1 * mean).max() < 1e-5
    assert rel_max(host(rv), 0.9 + 0.1 * yf.var(axis=0) * m / (m - 1)) < 1e-4


def test_maxpool_matches_oracle(orc):
    from renaissance_b200 import ops
    rng = np.random.default_rng(5)
    x = np.round(rng.standard_normal((3, 8, 6, 16)) * 2).astype(np.float16) / 2     # many ties
    y_ref, am_ref = orc.maxpool2x2_fwd(x)
    y, am = ops.maxpool2x2_fwd(dev(x))
    assert np.array_equal(host(y), y_ref) and np.array_equal(host(am), am_ref)       # bit-exact, argmax included
    dy = rng.standard_normal(y_ref.shape).astype(np.float16)
    dx = torch.full(x.shape, 9.0, dtype=torch.float16, device="cuda")
    ops.maxpool2x2_bwd(dev(dy), am, dx)
    assert np.array_equal(host(dx), orc.maxpool2x2_bwd(dy, am_ref, x.shape))


@pytest.mark.parametrize("n,h,w,c", [(2, 8, 6, 16), (3, 14, 14, 64), (1, 4, 4, 520), (5, 28, 28, 256)])
def test_pool_fused_into_block_forward_and_backward(orc, n, h, w, c):
    """The 2x2 max pool fused into the block's BN kernels: forward equals bn_apply_relu_mask followed
    by maxpool2x2_fwd bit for bit; backward equals maxpool2x2_bwd followed by the BN+ReLU backward
    (oracle) to the usual tolerances."""
    from renaissance_b200 import ops
    rng = np.random.default_rng(n * 3 + c)
    co = (rng.standard_normal((n, h, w, c)) * 1.2 + 0.1).astype(np.float16)
    co[0, :2, :2, :8] = 0.5                                   # ties inside a window: first maximum must win
    gamma = (1 + 0.2 * rng.standard_normal(c)).astype(np.float32)
    cf = co.astype(np.float32).reshape(-1, c)
    mean = cf.mean(axis=0).astype(np.float32)
    inv = (1.0 / np.sqrt(cf.var(axis=0) + 1e-5)).astype(np.float32)
    es = (gamma * inv).astype(np.float32)
    eb = (0.1 - mean * es).astype(np.float32)
    cod, esd, ebd = dev(co), dev(es), dev(eb)
    relu, bits = ops.bn_apply_relu_mask(cod, esd, ebd)
    pool_ref, am_ref = ops.maxpool2x2_fwd(relu)
    pool, am, bits2 = ops.bn_apply_relu_mask_pool(cod, esd, ebd)
    torch.cuda.synchronize()
    assert torch.equal(bits, bits2) and torch.equal(pool, pool_ref) and torch.equal(am, am_ref)
    # optional full-resolution output
    relu2 = torch.empty_like(relu)
    ops.bn_apply_relu_mask_pool(cod, esd, ebd, relu_out=relu2)
    assert torch.equal(relu2, relu)
    # backward
    dyp = rng.standard_normal((n, h // 2, w // 2, c)).astype(np.float16)
    dy_full = orc.maxpool2x2_bwd(dyp, host(am), co.shape)
    ref_dx, ref_dg, ref_db = orc.bnrelu_bwd_amp(dy_full, host(bits), co, gamma, mean, inv)
    dconv, dg, db = ops.bnrelu_pool_bwd(dev(dyp), am, bits, cod, dev(gamma), dev(mean), dev(inv))
    torch.cuda.synchronize()
    assert rel_max(host(dg), ref_dg) < 1e-4 and rel_max(host(db), ref_db) < 1e-4
    assert rel_l2(host(dconv).astype(np.float32), ref_dx.astype(np.float32)) < 2e-3
    d2, dg2, db2 = ops.bnrelu_pool_bwd(dev(dyp), am, bits, cod, dev(gamma), dev(mean), dev(inv))
    assert torch.equal(dg, dg2) and torch.equal(db, db2) and torch.equal(dconv, d2)      # reproducible


def test_sgd_momentum_and_nonfinite_guard(orc):
    from renaissance_b200 import ops
    rng = np.random.default_rng(6)
    n = 10007
    w = rng.standard_normal(n).astype(np.float32)
    g = (rng.standard_normal(n) * 1024).astype(np.float32)
    m = rng.standard_normal(n).astype(np.float32)
    w_ref, m_ref = orc.momentum(w, g, m, lr=0.1, wd=5e-4, beta=0.9, scaling=1024.0)
    pad = (-n) % 4
    wd_, gd, md = (torch.zeros(n + pad, device="cuda") for _ in range(3))
    wd_[:n], gd[:n], md[:n] = dev(w), dev(g), dev(m)
    w16 = torch.zeros(n + pad, dtype=torch.float16, device="cuda")
    scaling = torch.tensor([1024.0], device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.check_nonfinite(gd, flag)
    assert int(flag) == 0
    ops.sgd_momentum(wd_, gd, md, w16, 0.1, 5e-4, 0.9, scaling=scaling, skip_flag=flag)
    assert np.abs(host(wd_[:n]) - w_ref).max() < 1e-6 and np.abs(host(md[:n]) - m_ref).max() < 1e-6
    assert np.array_equal(host(w16[:n]), host(wd_[:n]).astype(np.float16))
    # a non-finite gradient raises the flag and the update is skipped (optimizer_op.cu:28)
    gd[17] = float("inf")
    ops.check_nonfinite(gd, flag)
    assert int(flag) == 1
    before = wd_.clone()
    ops.sgd_momentum(wd_, gd, md, w16, 0.1, 5e-4, 0.9, scaling=scaling, skip_flag=flag)
    assert torch.equal(wd_, before)


def test_whole_step_matches_oracle(orc):
    """One step of the GPU driver against the oracle's step.

    (1) Every block backward inside the chain is checked on ITS OWN inputs: a hook grabs
    the upstream gradient and the block input the driver hands to CBR_AMP_BWD, the oracle
    runs the same block on them, and dW / dgamma / dbeta / dX must agree to half
    precision.  This covers the wiring (in-place dX, pooling, first-layer variant).
    (2) End to end the two paths see slightly different activations (half rounding flips
    a few mask bits, 0.2 % at the deepest block), which the batch-norm backward of tiny
    4-image batches amplifies, so the end-to-end comparison is loose: loss within 1 %,
    forward activations within 1 %, classifier gradient within 3 %."""
    from oracle import vgg16bn_cpu as cpu
    from renaissance_b200 import ops
    from renaissance_b200.vgg16bn import Vgg16BnTrainer
    image, batch, classes = 64, 4, 1000
    params = cpu.init_params(seed=7, image=image, classes=classes, fc_width=256)
    img, labels = cpu.synthetic_batch(8, batch, image, classes)
    tr = Vgg16BnTrainer(batch=batch, image=image, classes=classes, lr=0.05, momentum=0.9, weight_decay=5e-4,
                        loss_scale=1024.0, dropout=0.0, fc_width=256, bucket_mb=1.0)
    tr.load_params(params)
    tr.images[0].copy_(torch.from_numpy(img))
    tr.labels[0].copy_(torch.from_numpy(labels))
    grabbed = {}

    def hook(L, dy, x):
        b = L.buf
        dy_h = host(dy).copy()
        if L.pool_after:        # the driver hands the pooled gradient + argmax to the block: unpool for the oracle
            dy_h = orc.maxpool2x2_bwd(dy_h, host(b["argmax"]), tuple(b["conv_out"].shape))
        grabbed[L.idx] = dict(dy=dy_h, x=host(x).copy(), conv_out=host(b["conv_out"]).copy(),
                              mask=host(b["mask"]).copy(), mean=host(b["saved_mean"]).copy(),
                              inv=host(b["saved_inv_std"]).copy())

    tr.debug_hook = hook
    w16_before = tr.w16.clone()
    loss = tr.step(0)
    ops.device_status()
    w_old = cpu.init_params(seed=7, image=image, classes=classes, fc_width=256)
    # (1) block by block on the driver's own tensors
    for L in tr.convs:
        g = grabbed[L.idx]
        w16 = host(tr.view(w16_before, L.w))
        ref = orc.cbr_bwd_amp(g["dy"], w16, w_old["convs"][L.idx]["gamma"], g["mean"], g["inv"], g["mask"], g["x"],
                              g["conv_out"], first_layer=(L.idx == 0))
        assert rel_l2(host(tr.half_grad(L.w)).astype(np.float32), ref["dw"].astype(np.float32)) < 3e-3, L.idx
        assert rel_max(host(tr.view(tr.g32, L.gamma)), ref["dgamma"]) < 1e-3, L.idx
        assert rel_max(host(tr.view(tr.g32, L.beta)), ref["dbeta"]) < 1e-3, L.idx
        if L.idx > 0:
            prev = tr.convs[L.idx - 1]
            dx_buf = prev.buf["pool_out"] if prev.pool_after else None
            if dx_buf is not None:          # not yet overwritten by the next stage
                assert rel_l2(host(dx_buf).astype(np.float32), ref["dx"].astype(np.float32)) < 3e-3, L.idx
    # (2) end to end
    ref = cpu.step(params, img, labels, lr=0.05, momentum=0.9, weight_decay=5e-4, loss_scale=1024.0)
    assert abs(float(loss) - ref["loss"]) < 1e-2 * abs(ref["loss"])
    assert rel_l2(host(tr.logits).astype(np.float32), ref["logits"].astype(np.float32)) < 2e-2
    assert rel_l2(host(tr.view(tr.g32, tr.fc[2]["w"])), ref["grads"]["fcs"][2]["w"]) < 3e-2
    # the optimizer moved the master weights the way the oracle's did, to the accuracy of the gradients
    got = tr.params()
    for i in (12, 0):
        upd = got["convs"][i]["w"] - w_old["convs"][i]["w"]
        upd_ref = params["convs"][i]["w"] - w_old["convs"][i]["w"]
        assert rel_l2(upd, upd_ref) < 0.35
    # the half working copy follows the master weights
    assert torch.equal(tr.w16, tr.w32.half())


def test_nesterov_plain_sgd_clip_and_loss_scale_backoff(orc):
    """The rest of the gradient post-processing chain (optimizer_op.cu:22-38, 68-93; check_op.cu:54-79;
    grad_scaling_op.cu:15-22) against the oracle's restatements."""
    from renaissance_b200 import ops
    rng = np.random.default_rng(11)
    n = 100003                                            # not a multiple of 4: the scalar tail runs too
    w = rng.standard_normal(n).astype(np.float32)
    g = (rng.standard_normal(n) * 1024).astype(np.float32)
    m = rng.standard_normal(n).astype(np.float32)
    scaling = torch.tensor([1024.0], device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    # Nesterov
    wd_, gd, md = dev(w), dev(g), dev(m)
    w16 = torch.empty(n, dtype=torch.float16, device="cuda")
    ops.sgd_nesterov(wd_, gd, md, w16, 0.05, 5e-4, 0.9, scaling=scaling, skip_flag=flag)
    w_ref, m_ref = orc.nesterov(w, g, m, 0.05, 5e-4, 0.9, 1024.0)
    assert np.abs(host(wd_) - w_ref).max() < 1e-6 and np.abs(host(md) - m_ref).max() < 1e-6
    assert torch.equal(w16, wd_.half())
    # plain SGD
    wd_ = dev(w)
    ops.sgd_plain(wd_, gd, None, 0.05, 5e-4, scaling=scaling, skip_flag=flag)
    assert np.abs(host(wd_) - orc.sgd(w, g, 0.05, 5e-4, 1024.0)).max() < 1e-6
    # NaN check with clipping: NaN flagged and kept, infinities and large values clamped, the rest untouched
    gc = g.copy()
    gc[5], gc[77], gc[1000], gc[n - 1] = np.nan, np.inf, -np.inf, 5000.0
    gcd = dev(gc)
    ops.check_nan_and_clip(gcd, 2048.0, flag)
    ref, ref_flag = orc.check_nan_and_clip(gc, 2048.0)
    got = host(gcd)
    assert int(flag) == 1 == ref_flag and np.isnan(got[5])
    assert np.array_equal(np.delete(got, 5), np.delete(ref, 5))
    clean = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.check_nan_and_clip(dev(g), 1e9, clean)
    assert int(clean) == 0
    # the optimizers skip a flagged step
    before = wd_.clone()
    ops.sgd_nesterov(wd_, gd, md, None, 0.05, 5e-4, 0.9, scaling=scaling, skip_flag=flag)
    ops.sgd_plain(wd_, gd, None, 0.05, 5e-4, scaling=scaling, skip_flag=flag)
    assert torch.equal(wd_, before)
    # loss-scale back-off: halves on a flagged step, stops at 1, leaves a clean step alone
    ops.grad_scaling(flag, scaling)
    assert float(scaling) == 512.0 == orc.grad_scaling(1, 1024.0) and int(flag) == 1
    ops.grad_scaling(clean, scaling)
    assert float(scaling) == 512.0
    low = torch.tensor([1.5], device="cuda")
    ops.grad_scaling(flag, low, clear_flag=True)
    assert float(low) == 1.0 == orc.grad_scaling(1, 1.5) and int(flag) == 0
