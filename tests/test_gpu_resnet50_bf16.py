"""The ResNet-50 bf16 configuration at the level the hot path reaches it: every distinct convolution of the
network (the reference lists them in scripts/resnet50_conv.json as kernel, in/out channels, in/out extent,
stride, padding) has its data and weight gradients checked against the CPU oracle on bfloat16 tensors, and
the BN+ReLU backward is checked on bfloat16 activations of the network's shapes.  The reference has no
backend for this configuration, so the oracle (float arithmetic on the bf16-rounded inputs) is the only
reference; the batch is 2 so that it finishes in seconds."""
import numpy as np
import pytest
import torch

from conftest import rel_l2, rel_max
from gpu_util import dev, host

pytestmark = pytest.mark.gpu

# kernel, in channels, out channels, input extent, output extent, stride, padding
RESNET50_CONVS = [
    (7, 4, 64, 224, 112, 2, 3),
    (1, 64, 64, 56, 56, 1, 0), (3, 64, 64, 56, 56, 1, 1), (1, 64, 256, 56, 56, 1, 0), (1, 256, 64, 56, 56, 1, 0),
    (1, 256, 128, 56, 56, 1, 0), (1, 256, 512, 56, 28, 2, 0), (3, 128, 128, 56, 28, 2, 1),
    (1, 128, 512, 28, 28, 1, 0), (1, 512, 128, 28, 28, 1, 0), (3, 128, 128, 28, 28, 1, 1),
    (1, 512, 256, 28, 28, 1, 0), (1, 512, 1024, 28, 14, 2, 0), (3, 256, 256, 28, 14, 2, 1),
    (1, 256, 1024, 14, 14, 1, 0), (1, 1024, 256, 14, 14, 1, 0), (3, 256, 256, 14, 14, 1, 1),
    (1, 1024, 512, 14, 14, 1, 0), (1, 1024, 2048, 14, 7, 2, 0), (3, 512, 512, 14, 7, 2, 1),
    (1, 512, 2048, 7, 7, 1, 0), (1, 2048, 512, 7, 7, 1, 0), (3, 512, 512, 7, 7, 1, 1),
]


def bf16_round(a):
    """float32 array with every value rounded to the nearest bfloat16."""
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).bfloat16().float().numpy()


def dev_bf16(a):
    return dev(a).bfloat16()


def host_f32(t):
    return host(t.float())


@pytest.mark.parametrize("r,c,k,h,oh,stride,pad", RESNET50_CONVS)
def test_conv_gradients_bf16_match_oracle(orc, r, c, k, h, oh, stride, pad):
    from renaissance_b200 import ops
    n = 2
    rng = np.random.default_rng(r * 1000 + c + k + h)
    x = bf16_round(rng.standard_normal((n, h, h, c)))
    wt = bf16_round(rng.standard_normal((k, r, r, c)) * np.sqrt(2.0 / (r * r * c)))
    dy = bf16_round(rng.standard_normal((n, oh, oh, k)))
    g = ops.ConvGeometry(n, h, h, c, k, r, r, pad, stride, dtype=torch.bfloat16)
    assert (g.oh, g.ow) == (oh, oh)
    # every layer runs on the tcgen05 kernels: the stride-2 ones through the stride-1 kernel and a resampling
    # pass, the 7x7 stem lowered to rows (its data gradient, which no network needs, on the direct kernel)
    assert ops.conv_uses_tensor_cores(g, "dgrad") == (r != 7)
    assert ops.conv_uses_tensor_cores(g, "wgrad")
    ref_dw = orc.conv_wgrad(dy, x, wt.shape, pad=pad, stride=stride)
    ref_dx = orc.conv_dgrad(dy, wt, x.shape, pad=pad, stride=stride)
    dw = ops.conv_wgrad(g, dev_bf16(dy), dev_bf16(x))
    dx = ops.conv_dgrad(g, dev_bf16(dy), dev_bf16(wt))
    ops.device_status()
    assert dw.dtype == torch.bfloat16 and dx.dtype == torch.bfloat16
    # 2e-2 relative L2 is the stated bound for 16-bit gradients; rounding the result to bf16 (8 significant
    # bits) alone gives about 2e-3
    assert rel_l2(host_f32(dw), ref_dw) < 2e-2 and rel_l2(host_f32(dx), ref_dx) < 2e-2
    assert rel_l2(host_f32(dw), ref_dw) < 4e-3 and rel_l2(host_f32(dx), ref_dx) < 4e-3


@pytest.mark.parametrize("m,c", [(2 * 112 * 112, 64), (2 * 56 * 56, 256), (2 * 28 * 28, 512), (2 * 14 * 14, 1024),
                                 (2 * 7 * 7, 2048), (33, 8)])
def test_bnrelu_bwd_bf16_matches_oracle(orc, m, c):
    from renaissance_b200 import ops
    rng = np.random.default_rng(m + c)
    dy = bf16_round(rng.standard_normal((m, c)))
    x = bf16_round(rng.standard_normal((m, c)) * 1.5 + 0.3)
    mask = (rng.random((m, c)) < 0.5).astype(np.int8)
    bits = orc.mask_pack(mask)
    gamma = (1.0 + 0.2 * rng.standard_normal(c)).astype(np.float32)
    mean = x.mean(axis=0).astype(np.float32)
    inv_std = (1.0 / np.sqrt(x.var(axis=0) + 1e-5)).astype(np.float32)
    # oracle: ReLU backward through the mask, then the float BN backward (double accumulators)
    dy_m = dy * mask.astype(np.float32)
    ref = orc.bn_bwd(dy_m, x, gamma, mean, inv_std)
    ref_dx, ref_dg, ref_db = ref[0], ref[1], ref[2]
    dconv, dg, db = ops.bnrelu_bwd(dev_bf16(dy), dev(bits), dev_bf16(x), dev(gamma), dev(mean), dev(inv_std))
    torch.cuda.synchronize()
    assert dconv.dtype == torch.bfloat16
    assert rel_max(host(dg), ref_dg) < 1e-4 and rel_max(host(db), ref_db) < 1e-4
    assert rel_l2(host_f32(dconv), ref_dx) < 2e-2
    assert rel_l2(host_f32(dconv), ref_dx) < 4e-3


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_bn_backward_without_relu_matches_oracle(orc, dtype):
    """mask_bits = NULL: the BN of a residual block's shortcut has no ReLU behind it."""
    from renaissance_b200 import ops
    m, c = 2 * 28 * 28, 512
    rng = np.random.default_rng(3)
    rnd = bf16_round if dtype == torch.bfloat16 else (lambda a: a.astype(np.float16).astype(np.float32))
    dy, x = rnd(rng.standard_normal((m, c))), rnd(rng.standard_normal((m, c)) * 1.5 + 0.3)
    gamma = (1.0 + 0.2 * rng.standard_normal(c)).astype(np.float32)
    mean = x.mean(axis=0).astype(np.float32)
    inv_std = (1.0 / np.sqrt(x.var(axis=0) + 1e-5)).astype(np.float32)
    ref_dx, ref_dg, ref_db = orc.bn_bwd(dy, x, gamma, mean, inv_std)
    dconv, dg, db = ops.bnrelu_bwd(dev(dy).to(dtype), None, dev(x).to(dtype), dev(gamma), dev(mean), dev(inv_std))
    torch.cuda.synchronize()
    assert rel_max(host(dg), ref_dg) < 1e-4 and rel_max(host(db), ref_db) < 1e-4
    assert rel_l2(host_f32(dconv), ref_dx) < (4e-3 if dtype == torch.bfloat16 else 2e-3)
    # and it equals the masked operator with an all-ones mask, bit for bit
    ones = torch.full((m * c // 8,), 255, dtype=torch.uint8, device="cuda")
    d2, dg2, db2 = ops.bnrelu_bwd(dev(dy).to(dtype), ones, dev(x).to(dtype), dev(gamma), dev(mean), dev(inv_std))
    assert torch.equal(dconv, d2) and torch.equal(dg, dg2) and torch.equal(db, db2)


@pytest.mark.parametrize("n,h,w,c,k", [(2, 8, 8, 64, 64), (3, 7, 5, 64, 128), (2, 14, 14, 128, 256),
                                       (1, 9, 33, 64, 512), (5, 12, 20, 256, 64), (2, 28, 28, 128, 128),
                                       (4, 14, 14, 512, 512)])
def test_tensor_core_kernels_bf16_match_oracle(orc, n, h, w, c, k):
    """Every tcgen05 kernel variant (pixels on M with 256-filter tiles, pixels on N with 64 / 128 filters, both
    weight-gradient kernels, the statistics epilogue) on bfloat16 operands."""
    from renaissance_b200 import ops
    rng = np.random.default_rng(n + 3 * h + c)
    x = bf16_round(rng.standard_normal((n, h, w, c)))
    wt = bf16_round(rng.standard_normal((k, 3, 3, c)) * np.sqrt(2.0 / (9 * c)))
    dy = bf16_round(rng.standard_normal((n, h, w, k)))
    g = ops.ConvGeometry(n, h, w, c, k, dtype=torch.bfloat16)
    for which in ("wgrad", "dgrad", "fprop"):
        assert ops.conv_uses_tensor_cores(g, which)
    dw = ops.conv_wgrad(g, dev_bf16(dy), dev_bf16(x))
    dx = ops.conv_dgrad(g, dev_bf16(dy), dev_bf16(wt))
    y = ops.conv_fprop(g, dev_bf16(x), dev_bf16(wt))
    gamma, beta = np.ones(k, np.float32), np.zeros(k, np.float32)
    y2, st = ops.conv_fprop_bn_stats(g, dev_bf16(x), dev_bf16(wt), dev(gamma), dev(beta), want_sums=True)
    ops.device_status()
    ref_y = orc.conv_fwd(x, wt)
    assert rel_l2(host_f32(dx), orc.conv_dgrad(dy, wt, x.shape)) < 4e-3
    assert rel_l2(host_f32(dw), orc.conv_wgrad(dy, x, wt.shape)) < 4e-3
    assert rel_l2(host_f32(y), ref_y) < 4e-3
    assert torch.equal(y, y2)
    # the statistics are those of the rounded (bf16) output
    yr = host_f32(y).reshape(-1, k).astype(np.float64)
    assert rel_max(host(st["sum"]), yr.sum(axis=0)) < 1e-4
    assert rel_max(host(st["sqsum"]), (yr * yr).sum(axis=0)) < 1e-4


def test_bf16_and_half_kernels_agree_on_values_both_types_hold(orc):
    """Values that are exact in both 16-bit types (small integers / 4) must give the same gradients through
    the bf16 and the half kernels up to the rounding of the result."""
    from renaissance_b200 import ops
    n, h, c, k = 2, 12, 16, 24
    rng = np.random.default_rng(5)
    x = rng.integers(-8, 9, (n, h, h, c)).astype(np.float32) / 4
    wt = rng.integers(-8, 9, (k, 3, 3, c)).astype(np.float32) / 8
    dy = rng.integers(-8, 9, (n, h, h, k)).astype(np.float32) / 4
    out = {}
    for dt in (torch.float16, torch.bfloat16):
        g = ops.ConvGeometry(n, h, h, c, k, dtype=dt)
        out[dt] = (ops.conv_wgrad(g, dev(dy).to(dt), dev(x).to(dt)).float(),
                   ops.conv_dgrad(g, dev(dy).to(dt), dev(wt).to(dt)).float())
    torch.cuda.synchronize()
    for a, b in zip(out[torch.float16], out[torch.bfloat16]):
        assert rel_l2(host(b), host(a)) < 4e-3


def _bn_stats(t):
    """saved mean / inv_std of a stored [n,h,w,c] tensor (biased variance, eps 1e-5)."""
    f = t.reshape(-1, t.shape[-1]).astype(np.float64)
    return f.mean(axis=0).astype(np.float32), (1.0 / np.sqrt(f.var(axis=0) + 1e-5)).astype(np.float32)


def _bn_relu_fwd(t, gamma, beta, relu=True):
    mean, inv = _bn_stats(t)
    y = bf16_round((t - mean) * inv * gamma + beta)
    if not relu:
        return y, mean, inv, None
    mask = (y > 0).astype(np.int8)
    return y * mask, mean, inv, mask


@pytest.mark.parametrize("cin,mid,cout,stride", [(256, 64, 256, 1), (256, 128, 512, 2)])
def test_bottleneck_backward_composed_from_the_entry_points(orc, cin, mid, cout, stride):
    """A ResNet-50 bottleneck (1x1 -> 3x3 -> 1x1, BN after each, ReLU after the first two and after the join;
    identity shortcut, or 1x1 stride-2 conv + BN when the block changes resolution) run backward through the
    library's entry points on bfloat16 tensors.  Every operator is checked against the oracle on the inputs it
    actually received (per-operator tolerances), and the block's dx against the oracle's whole chain."""
    from renaissance_b200 import ops
    bf = torch.bfloat16
    n, h = 2, 14
    oh = (h - 1) // stride + 1
    rng = np.random.default_rng(cin + stride)
    he = lambda k, r, c: bf16_round(rng.standard_normal((k, r, r, c)) * np.sqrt(2.0 / (r * r * c)))   # noqa: E731
    gb = lambda c: ((1.0 + 0.2 * rng.standard_normal(c)).astype(np.float32),                         # noqa: E731
                    (0.2 * rng.standard_normal(c)).astype(np.float32))
    x0 = bf16_round(np.maximum(rng.standard_normal((n, h, h, cin)), 0))
    w1, w2, w3 = he(mid, 1, cin), he(mid, 3, mid), he(cout, 1, mid)
    (g1, b1), (g2, b2), (g3, b3) = gb(mid), gb(mid), gb(cout)
    # forward by the oracle, every stored tensor rounded to bf16
    c1 = bf16_round(orc.conv_fwd(x0, w1, pad=0))
    a1, m1, i1, k1 = _bn_relu_fwd(c1, g1, b1)
    c2 = bf16_round(orc.conv_fwd(a1, w2, pad=1, stride=stride))
    a2, m2, i2, k2 = _bn_relu_fwd(c2, g2, b2)
    c3 = bf16_round(orc.conv_fwd(a2, w3, pad=0))
    y3, m3, i3, _ = _bn_relu_fwd(c3, g3, b3, relu=False)
    if stride == 1:
        sc = x0
    else:
        wd = he(cout, 1, cin)
        gd, bd = gb(cout)
        cd = bf16_round(orc.conv_fwd(x0, wd, pad=0, stride=stride))
        sc, md, idv, _ = _bn_relu_fwd(cd, gd, bd, relu=False)
    dout = bf16_round(rng.standard_normal((n, oh, oh, cout)))

    D = dev_bf16
    bits = lambda k: dev(orc.mask_pack(k.reshape(-1, k.shape[-1])))   # noqa: E731
    # the join forward: relu(y3 + shortcut) and its mask, bit-exact against numpy
    out_ref = bf16_round(y3 + sc)
    kout = (out_ref > 0).astype(np.int8)
    out_gpu, mout = ops.add_relu_mask(D(y3), D(sc))
    assert np.array_equal(host_f32(out_gpu), out_ref * kout)
    assert np.array_equal(host(mout), orc.mask_pack(kout.reshape(-1, cout)))

    geo1 = ops.ConvGeometry(n, h, h, cin, mid, 1, 1, 0, 1, dtype=bf)
    geo2 = ops.ConvGeometry(n, h, h, mid, mid, 3, 3, 1, stride, dtype=bf)
    geo3 = ops.ConvGeometry(n, oh, oh, mid, cout, 1, 1, 0, 1, dtype=bf)

    def check_bn(dy_t, mask_np, conv_np, gamma, mean, inv, got):
        dy_np = host_f32(dy_t)
        if mask_np is not None:
            dy_np = dy_np * mask_np
        rdx, rdg, rdb = orc.bn_bwd(dy_np.reshape(-1, dy_np.shape[-1]), conv_np.reshape(-1, conv_np.shape[-1]),
                                   gamma, mean, inv)
        dconv, dg, db = got
        assert rel_max(host(dg), rdg) < 1e-4 and rel_max(host(db), rdb) < 1e-4
        assert rel_l2(host_f32(dconv).reshape(rdx.shape), rdx) < 4e-3

    def check_conv(geo, dconv_t, act_np, w_np, dw, dx):
        dc = host_f32(dconv_t)
        assert rel_l2(host_f32(dw), orc.conv_wgrad(dc, act_np, w_np.shape, pad=geo.pad, stride=geo.stride)) < 4e-3
        if dx is not None:
            assert rel_l2(host_f32(dx), orc.conv_dgrad(dc, w_np, act_np.shape, pad=geo.pad, stride=geo.stride)) < 4e-3

    g = ops.relu_mask_bwd(D(dout), mout)
    assert np.array_equal(host_f32(g), dout * kout)
    r3 = ops.bnrelu_bwd(g, None, D(c3), dev(g3), dev(m3), dev(i3))
    check_bn(g, None, c3, g3, m3, i3, r3)
    dw3, da2 = ops.conv_wgrad(geo3, r3[0], D(a2)), ops.conv_dgrad(geo3, r3[0], D(w3))
    check_conv(geo3, r3[0], a2, w3, dw3, da2)
    r2 = ops.bnrelu_bwd(da2, bits(k2), D(c2), dev(g2), dev(m2), dev(i2))
    check_bn(da2, k2, c2, g2, m2, i2, r2)
    dw2, da1 = ops.conv_wgrad(geo2, r2[0], D(a1)), ops.conv_dgrad(geo2, r2[0], D(w2))
    check_conv(geo2, r2[0], a1, w2, dw2, da1)
    r1 = ops.bnrelu_bwd(da1, bits(k1), D(c1), dev(g1), dev(m1), dev(i1))
    check_bn(da1, k1, c1, g1, m1, i1, r1)
    dw1, dx_main = ops.conv_wgrad(geo1, r1[0], D(x0)), ops.conv_dgrad(geo1, r1[0], D(w1))
    check_conv(geo1, r1[0], x0, w1, dw1, dx_main)
    if stride == 1:
        dx_sc = g
    else:
        geod = ops.ConvGeometry(n, h, h, cin, cout, 1, 1, 0, stride, dtype=bf)
        rd = ops.bnrelu_bwd(g, None, D(cd), dev(gd), dev(md), dev(idv))
        check_bn(g, None, cd, gd, md, idv, rd)
        dwd, dx_sc = ops.conv_wgrad(geod, rd[0], D(x0)), ops.conv_dgrad(geod, rd[0], D(wd))
        check_conv(geod, rd[0], x0, wd, dwd, dx_sc)
    dx = ops.add16(dx_main, dx_sc)
    ops.device_status()
    assert np.array_equal(host_f32(dx), bf16_round(host_f32(dx_main) + host_f32(dx_sc)))

    # the whole chain by the oracle (bf16 rounding where a tensor is stored): the block's dx within the 16-bit bound
    def o_bn(dy_np, mask_np, conv_np, gamma, mean, inv):
        if mask_np is not None:
            dy_np = dy_np * mask_np
        rdx, _, _ = orc.bn_bwd(dy_np.reshape(-1, dy_np.shape[-1]), conv_np.reshape(-1, conv_np.shape[-1]), gamma,
                               mean, inv)
        return bf16_round(rdx.reshape(conv_np.shape))

    og = dout * kout
    o3 = o_bn(og, None, c3, g3, m3, i3)
    oa2 = bf16_round(orc.conv_dgrad(o3, w3, a2.shape, pad=0))
    o2 = o_bn(oa2, k2, c2, g2, m2, i2)
    oa1 = bf16_round(orc.conv_dgrad(o2, w2, a1.shape, pad=1, stride=stride))
    o1 = o_bn(oa1, k1, c1, g1, m1, i1)
    odx = bf16_round(orc.conv_dgrad(o1, w1, x0.shape, pad=0))
    if stride == 1:
        osc = og
    else:
        osc = bf16_round(orc.conv_dgrad(o_bn(og, None, cd, gd, md, idv), wd, x0.shape, pad=0, stride=stride))
    assert rel_l2(host_f32(dx), bf16_round(odx + osc)) < 2e-2


@pytest.mark.parametrize("batch,classes,ls", [(256, 1000, 0.0), (64, 1000, 0.1), (33, 2048, 0.0), (7, 8, 0.1)])
def test_softmax_ce_fused_on_bf16_logits(orc, batch, classes, ls):
    """The loss head of a bfloat16 network.  The logits are multiples of 1/8 in [-6, 6], exact in half and in
    bfloat16 alike, so the oracle's AMP operator (half logits) is the reference for loss and gradient; the
    gradient is rounded to bfloat16 here and to half there."""
    from renaissance_b200 import _lib, ops
    rng = np.random.default_rng(batch + classes)
    z = rng.integers(-48, 49, (batch, classes)).astype(np.float32) / 8
    labels = rng.integers(0, classes, size=batch).astype(np.int32)
    ref = orc.softmax_ce_amp(z.astype(np.float16), labels, scaling=1024.0, ls=ls)
    sc = torch.tensor([1024.0], device="cuda")
    lsd = torch.tensor([ls], device="cuda")
    zd, ld = dev(z).bfloat16(), dev(labels)
    assert np.array_equal(host_f32(zd), z)
    out = ops.softmax_ce_amp_fused(zd, ld, sc, lsd)
    torch.cuda.synchronize()
    assert out["dlogits"].dtype == torch.bfloat16
    assert abs(float(out["loss"]) - ref["loss"]) < 2e-5 * max(1.0, abs(ref["loss"]))
    assert np.allclose(host(out["loss_partial"]), ref["loss_partial"], rtol=1e-4, atol=1e-7)
    assert rel_l2(host_f32(out["dlogits"]), ref["dlogits"].astype(np.float32)) < 4e-3
    # the same call on the same values as half agrees to the two roundings
    half = ops.softmax_ce_amp_fused(dev(z).half(), ld, sc, lsd)
    assert rel_l2(host_f32(out["dlogits"]), host_f32(half["dlogits"])) < 4e-3
    assert abs(float(out["loss"]) - float(half["loss"])) < 1e-6 * max(1.0, abs(ref["loss"]))
    # longer rows are refused for bfloat16, loudly
    with pytest.raises(_lib.Trb200Error):
        ops.softmax_ce_amp_fused(torch.zeros((4, 4096), device="cuda", dtype=torch.bfloat16),
                                 torch.zeros(4, device="cuda", dtype=torch.int32), sc, lsd)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n,h,w,c,k,stride,pad", [(2, 112, 112, 64, 3, 2, 1), (3, 9, 7, 16, 3, 2, 1),
                                                  (2, 8, 8, 8, 2, 2, 0), (1, 11, 13, 24, 5, 3, 2), (2, 6, 6, 8, 3, 1, 1)])
def test_general_max_pool_matches_oracle(orc, dtype, n, h, w, c, k, stride, pad):
    """ResNet's 3x3 stride-2 pool after the stem, and other windows: outputs and argmax bytes bit for bit, the
    backward (a float gather per input pixel) to the rounding of the result."""
    from renaissance_b200 import ops
    rng = np.random.default_rng(h * 7 + c + k)
    rnd = bf16_round if dtype == torch.bfloat16 else (lambda a: a.astype(np.float16).astype(np.float32))
    x = rnd(rng.standard_normal((n, h, w, c)))
    x[0, : min(h, 4), : min(w, 4), 0] = 1.0          # ties: the first maximum must win
    ref_y, ref_am = orc.maxpool_fwd(x, k, stride, pad)
    y, am = ops.maxpool_fwd(dev(x).to(dtype), k, stride, pad)
    torch.cuda.synchronize()
    assert np.array_equal(host_f32(y), ref_y)
    assert np.array_equal(host(am), ref_am)
    dy = rnd(rng.standard_normal(ref_y.shape))
    dx = ops.maxpool_bwd(dev(dy).to(dtype), am, x.shape, k, stride, pad)
    ref_dx = orc.maxpool_bwd(dy, ref_am, x.shape, k, stride, pad)
    assert np.array_equal(host_f32(dx), rnd(ref_dx))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n,h,w,c", [(4, 7, 7, 2048), (3, 5, 3, 8)])
def test_global_average_pool_matches_oracle(orc, dtype, n, h, w, c):
    from renaissance_b200 import ops
    rng = np.random.default_rng(h + c)
    rnd = bf16_round if dtype == torch.bfloat16 else (lambda a: a.astype(np.float16).astype(np.float32))
    x = rnd(rng.standard_normal((n, h, w, c)))
    y = ops.avgpool_global_fwd(dev(x).to(dtype))
    assert np.array_equal(host_f32(y), rnd(orc.avgpool_global_fwd(x)))
    dy = rnd(rng.standard_normal((n, c)))
    dx = ops.avgpool_global_bwd(dev(dy).to(dtype), h, w)
    assert np.array_equal(host_f32(dx), rnd(orc.avgpool_global_bwd(dy, h, w)))


@pytest.mark.parametrize("n,h,c,k,r,pad,stride", [(2, 28, 128, 128, 3, 1, 2), (2, 14, 256, 64, 1, 0, 1),
                                                  (3, 14, 64, 64, 3, 1, 1), (2, 15, 256, 512, 1, 0, 2)])
def test_block_backward_entry_point_on_resnet_blocks_bf16(orc, n, h, c, k, r, pad, stride):
    """trb200_cbr_bwd (BN+ReLU backward, weight gradient, data gradient in place over x, three streams) on the
    conv+BN+ReLU blocks a bottleneck is made of: 1x1, 3x3, and their stride-2 forms, bfloat16."""
    from renaissance_b200 import ops
    bf = torch.bfloat16
    rng = np.random.default_rng(h + c + k + r)
    oh = (h + 2 * pad - r) // stride + 1
    x = bf16_round(rng.standard_normal((n, h, h, c)))
    wt = bf16_round(rng.standard_normal((k, r, r, c)) * np.sqrt(2.0 / (r * r * c)))
    conv = bf16_round(orc.conv_fwd(x, wt, pad=pad, stride=stride))
    gamma = (1.0 + 0.2 * rng.standard_normal(k)).astype(np.float32)
    beta = (0.2 * rng.standard_normal(k)).astype(np.float32)
    _, mean, inv, mask = _bn_relu_fwd(conv, gamma, beta)
    dy = bf16_round(rng.standard_normal((n, oh, oh, k)))
    g = ops.ConvGeometry(n, h, h, c, k, r, r, pad, stride, dtype=bf)
    xd = dev_bf16(x)
    st = ops.BlockStreams.create()
    torch.cuda.synchronize()
    with torch.cuda.stream(st.bn):
        out = ops.cbr_amp_bwd(g, dev_bf16(dy), dev_bf16(wt), dev(gamma), dev(mean), dev(inv),
                              dev(orc.mask_pack(mask.reshape(-1, k))), xd, dev_bf16(conv), streams=st)
    torch.cuda.current_stream().wait_stream(st.bn)
    ops.device_status()
    assert out["dx"].data_ptr() == xd.data_ptr()          # in place over x, as in the reference
    rdx, rdg, rdb = orc.bn_bwd((dy * mask).reshape(-1, k), conv.reshape(-1, k), gamma, mean, inv)
    assert rel_max(host(out["dgamma"]), rdg) < 1e-4 and rel_max(host(out["dbeta"]), rdb) < 1e-4
    assert rel_l2(host_f32(out["dconv"]).reshape(rdx.shape), rdx) < 4e-3
    dconv = host_f32(out["dconv"])
    assert rel_l2(host_f32(out["dw"]), orc.conv_wgrad(dconv, x, wt.shape, pad=pad, stride=stride)) < 4e-3
    assert rel_l2(host_f32(out["dx"]), orc.conv_dgrad(dconv, wt, x.shape, pad=pad, stride=stride)) < 4e-3


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("relu", [True, False])
def test_bn_forward_stats_and_apply_either_type(orc, dtype, relu):
    """Batch statistics + apply on a conv output of either type: t = round(round(x*s) + b), bit for bit; ReLU and
    mask when asked for, the plain BN output otherwise (the BN in front of a residual join)."""
    from renaissance_b200 import ops
    m, c = 2 * 14 * 14, 256
    rng = np.random.default_rng(17)
    rnd = bf16_round if dtype == torch.bfloat16 else (lambda a: a.astype(np.float16).astype(np.float32))
    x = rnd(rng.standard_normal((m, c)) * 1.3 + 0.2)
    gamma = (1.0 + 0.2 * rng.standard_normal(c)).astype(np.float32)
    beta = (0.2 * rng.standard_normal(c)).astype(np.float32)
    st = ops.bn_stats_finalize(dev(x).to(dtype), dev(gamma), dev(beta), want_sums=True)
    x64 = x.astype(np.float64)
    assert rel_max(host(st["sum"]), x64.sum(axis=0)) < 1e-4
    assert rel_max(host(st["sqsum"]), (x64 * x64).sum(axis=0)) < 1e-4
    assert rel_max(host(st["saved_mean"]), x64.mean(axis=0)) < 1e-4
    assert rel_max(host(st["saved_inv_std"]), 1.0 / np.sqrt(x64.var(axis=0) + 1e-5)) < 1e-4
    es, eb = host(st["eq_scale"]), host(st["eq_bias"])
    t = rnd(rnd(x * es) + eb)                                  # float32 products and sums, as the kernel's
    out, bits = ops.bn_apply(dev(x).to(dtype), st["eq_scale"], st["eq_bias"], relu=relu)
    torch.cuda.synchronize()
    if relu:
        assert np.array_equal(host_f32(out), np.maximum(t, 0))
        assert np.array_equal(host(bits), orc.mask_pack((t > 0).astype(np.int8)))
    else:
        assert bits is None and np.array_equal(host_f32(out), t)
