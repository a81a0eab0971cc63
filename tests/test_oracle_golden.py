"""Pins the CPU oracle to the golden vectors (PyTorch recipes of the reference's
own test generators, see tests/golden/make_golden.py).  CPU only."""
import numpy as np
import pytest

from conftest import golden, rel_l2, rel_max


@pytest.mark.parametrize("name", ["conv_fp32_3x3_s1", "conv_fp32_3x3_s2", "conv_fp32_7x7_s2",
                                  "conv_fp16_3x3_s1"])
def test_conv_matches_golden(orc, name):
    g = golden(name)
    n, h, w, c, k, ker, stride, pad, _ = g["params"]
    y = orc.conv_fwd(g["x"], g["w"], pad=pad, stride=stride)
    dx = orc.conv_dgrad(g["dy"], g["w"], g["x"].shape, pad=pad, stride=stride)
    dw = orc.conv_wgrad(g["dy"], g["x"], g["w"].shape, pad=pad, stride=stride)
    # the reference's own threshold is MSE <= 1e-5 (tests/op/test_conv_fwd_bwd.cpp:366)
    for got, ref in ((y, g["y"]), (dx, g["dx"]), (dw, g["dw"])):
        assert np.mean((got - ref) ** 2) <= 1e-10
        assert rel_l2(got, ref) < 2e-6
    assert rel_max(y.sum(axis=(0, 1, 2)), g["ysum"]) < 1e-5
    assert rel_max((y ** 2).sum(axis=(0, 1, 2)), g["ysqsum"]) < 1e-5


@pytest.mark.parametrize("name", ["bn2d_fp32", "bn1d_fp32"])
def test_bn_matches_golden(orc, name):
    g = golden(name)
    c = int(g["params"][3])
    rm, rv = np.zeros(c, np.float32), np.ones(c, np.float32)
    y, mean, inv = orc.bn_fwd(g["x"], g["gamma"], g["beta"], rm, rv, float(g["eps"]), float(g["momentum"]))
    assert rel_l2(y, g["y"]) < 1e-6
    assert np.allclose(mean, g["saved_mean"], atol=1e-6)
    assert rel_max(inv, g["saved_inv_std"]) < 1e-6
    assert np.allclose(rm, g["running_mean"], atol=1e-6)
    assert rel_max(rv, g["running_var"]) < 1e-6
    dx, dg, db = orc.bn_bwd(g["dy"], g["x"], g["gamma"], mean, inv)
    assert rel_l2(dx, g["dx"]) < 1e-5
    assert rel_max(dg, g["dgamma"]) < 1e-5
    assert rel_max(db, g["dbeta"]) < 1e-5


@pytest.mark.parametrize("name", ["softmax_fp32_1000", "softmax_fp16_1000", "softmax_fp32_10"])
def test_softmax_cpu_operator_matches_golden(orc, name):
    g = golden(name)
    batch = int(g["params"][0])
    loss, inv, probs = orc.softmax_ce_fwd_cpu(g["logits"], g["labels"], scaling=1.0, ls=0.0)
    # reference thresholds: loss/probs MSE <= 1e-6 (tests/correction/test_softmax_ce.cpp:319-353)
    assert abs(loss - float(g["loss"])) < 2e-5
    assert inv == pytest.approx(1.0 / batch)
    assert np.abs(probs - g["probs"]).max() < 1e-6
    d = orc.softmax_ce_bwd(probs, g["labels"], scale=1.0 * inv, ls=0.0)
    assert np.abs(d - g["dlogits"]).max() < 1e-6
    assert np.array_equal(probs.argmax(axis=1).astype(np.int32), g["pred"])


def test_softmax_cpu_operator_accumulates_then_scales(orc):
    """*loss += ...; *loss *= scaling  (softmax_ce_op.cpp:152-155)."""
    g = golden("softmax_fp32_10")
    base, _, _ = orc.softmax_ce_fwd_cpu(g["logits"], g["labels"], scaling=1.0, ls=0.0)
    got, _, _ = orc.softmax_ce_fwd_cpu(g["logits"], g["labels"], scaling=4.0, ls=0.0, loss_init=0.5)
    assert got == pytest.approx((0.5 + base) * 4.0, rel=1e-6)


@pytest.mark.parametrize("name", ["softmax_fp16_1000", "softmax_fp16_ls"])
def test_softmax_amp_semantics_match_golden(orc, name):
    g = golden(name)
    batch, classes, _ = g["params"]
    ls, scaling = float(g["ls"]), float(g["scaling"])
    out = orc.softmax_ce_amp(g["logits"].astype(np.float16), g["labels"], scaling=scaling, ls=ls)
    # the GPU operator does not multiply the loss by `scaling` (softmax_ce_op.cu:171-173)
    assert abs(out["loss"] - float(g["loss"])) < 5e-5
    assert out["inv_scaling"] == pytest.approx(1.0 / batch)
    assert np.abs(out["probs"] - g["probs"]).max() < 1e-6
    # fp16 gradient: the reference allows MSE <= 1e-3 for fp16 d_logits; half rounding only here
    ref = g["dlogits"]
    assert rel_l2(out["dlogits"].astype(np.float32), ref) < 1e-3
    assert np.array_equal(out["probs"].argmax(axis=1).astype(np.int32), g["pred"])
    assert out["loss_partial"].sum() == pytest.approx(out["loss"], rel=1e-5)


@pytest.mark.parametrize("round_steps", [True, False])
@pytest.mark.parametrize("name", ["cbr_block_small", "cbr_block_first"])
def test_cbr_block_matches_golden(orc, name, round_steps):
    g = golden(name)
    first = bool(g["params"][5])
    fwd = orc.cbr_fwd_amp(g["x"], g["w"], g["gamma"], g["beta"], round_steps=round_steps)
    assert rel_l2(fwd["conv_out"].astype(np.float32), g["conv_out"]) < 1e-3
    assert np.allclose(fwd["saved_mean"], g["saved_mean"], atol=1e-5)
    assert rel_max(fwd["saved_inv_std"], g["saved_inv_std"]) < 1e-5
    assert rel_l2(fwd["relu_out"].astype(np.float32), g["relu_out"]) < 2e-3
    mask = orc.mask_unpack(fwd["mask_bits"], g["mask"].size).reshape(g["mask"].shape)
    # the golden mask comes from unrounded fp32 activations: only values that are
    # within half rounding of zero may differ
    assert (mask != g["mask"]).mean() < 2e-3
    # backward from the GOLDEN mask so that the comparison is like for like
    bits = orc.mask_pack(g["mask"])
    bwd = orc.cbr_bwd_amp(g["dy"], g["w"], g["gamma"], fwd["saved_mean"], fwd["saved_inv_std"],
                          bits, g["x"], fwd["conv_out"], first_layer=first)
    assert rel_max(bwd["dgamma"], g["dgamma"]) < 2e-3
    assert rel_max(bwd["dbeta"], g["dbeta"]) < 2e-3
    assert rel_l2(bwd["dw"].astype(np.float32), g["dw"]) < 5e-3
    if first:
        assert bwd["dx"] is None
    else:
        assert rel_l2(bwd["dx"].astype(np.float32), g["dx"]) < 5e-3


def test_cbr_fused_equals_unfused_chain(orc):
    """The reference's own CBR test compares the fused op with the Conv / BN / ReLU
    chain (tests/op/test_cbr_amp_bwd.cpp).  Same here, inside the oracle: the fused
    backward against relu_bwd -> bn_bwd -> conv_bwd on the same half inputs."""
    g = golden("cbr_block_small")
    fwd = orc.cbr_fwd_amp(g["x"], g["w"], g["gamma"], g["beta"])
    n_el = g["dy"].size
    mask = orc.mask_unpack(fwd["mask_bits"], n_el).reshape(g["dy"].shape)
    fused = orc.cbr_bwd_amp(g["dy"], g["w"], g["gamma"], fwd["saved_mean"], fwd["saved_inv_std"],
                            fwd["mask_bits"], g["x"], fwd["conv_out"])
    d_relu = orc.relu_bwd(g["dy"].astype(np.float32), mask)
    d_bn, dg, db = orc.bn_bwd(d_relu, fwd["conv_out"].astype(np.float32), g["gamma"],
                              fwd["saved_mean"], fwd["saved_inv_std"])
    d_bn16 = d_bn.astype(np.float16).astype(np.float32)
    # both paths of the reference's test hand back half tensors
    dx = orc.conv_dgrad(d_bn16, g["w"].astype(np.float32), g["x"].shape).astype(np.float16).astype(np.float32)
    dw = orc.conv_wgrad(d_bn16, g["x"].astype(np.float32), g["w"].shape).astype(np.float16).astype(np.float32)
    assert rel_max(fused["dgamma"], dg) < 1e-5
    assert rel_max(fused["dbeta"], db) < 1e-5
    # reference threshold: MSE <= 1e-6 between the two paths
    assert np.mean((fused["dx"].astype(np.float32) - dx) ** 2) <= 1e-6
    assert np.mean((fused["dw"].astype(np.float32) - dw) ** 2) <= 1e-6


def test_mask_bit_order(orc):
    """bit i%8 of byte i/8, least significant first (tests/op/cbr_amp_test_utils.hpp:115-145)."""
    m = np.zeros(24, np.int8)
    m[[0, 3, 9, 23]] = 1
    bits = orc.mask_pack(m)
    assert bits.tolist() == [0b00001001, 0b00000010, 0b10000000]
    assert np.array_equal(orc.mask_unpack(bits, 24), m)
    assert np.array_equal(bits, np.packbits(m.astype(np.uint8), bitorder="little"))


def _mlp_step(orc, x, labels, ws, bs, lr):
    acts = [x]
    h = x
    for li, (w, b) in enumerate(zip(ws, bs)):
        h = orc.fc_fwd(h, w, b)
        if li + 1 < len(ws):
            h, _ = orc.relu_fwd(h)
        acts.append(h)
    loss, inv, probs = orc.softmax_ce_fwd_cpu(acts[-1], labels)
    d = orc.softmax_ce_bwd(probs, labels, scale=inv)
    grads = []
    for li in reversed(range(len(ws))):
        dx, dw, db = orc.fc_bwd(d, ws[li], acts[li])
        grads.append((dw, db))
        if li > 0:
            d = orc.relu_bwd(dx, (acts[li] > 0).astype(np.int8))
    grads.reverse()
    new = [(orc.sgd(w, dw, lr), orc.sgd(b, db, lr)) for (w, b), (dw, db) in zip(zip(ws, bs), grads)]
    return loss, acts[-1], grads, new


def test_mlp_small_step_matches_golden(orc):
    g = golden("mlp_small")
    nl = len(g["sizes"]) - 1
    ws = [g[f"w{i}"] for i in range(nl)]
    bs = [np.zeros(w.shape[0], np.float32) for w in ws]
    loss, logits, grads, new = _mlp_step(orc, g["x"], g["labels"], ws, bs, float(g["lr"]))
    assert loss == pytest.approx(float(g["loss"]), abs=2e-6)
    assert np.abs(logits - g["logits"]).max() < 1e-5
    for i in range(nl):
        assert np.abs(grads[i][0] - g[f"dw{i}"]).max() < 1e-6
        assert np.abs(new[i][0] - g[f"w{i}_new"]).max() < 1e-6
        assert np.abs(new[i][1] - g[f"b{i}_new"]).max() < 1e-6


def test_mlp_config1_step_matches_golden(orc):
    """BASELINE.json configuration 1 (784-512-256-10, batch 128, SGD lr 0.1) on the oracle's
    restatement of the reference CPU backend; tensors rebuilt from the seed."""
    g = golden("mlp_config1")
    sizes, batch, seed = g["sizes"].tolist(), int(g["batch"]), int(g["seed"])
    rng = np.random.default_rng(seed)
    x = rng.random((batch, sizes[0]), dtype=np.float32)
    labels = rng.integers(0, sizes[-1], size=batch).astype(np.int32)
    ws = [(rng.standard_normal((o, i)) * np.sqrt(2.0 / i)).astype(np.float32)
          for i, o in zip(sizes[:-1], sizes[1:])]
    bs = [np.zeros(o, np.float32) for o in sizes[1:]]
    loss, logits, grads, new = _mlp_step(orc, x, labels, ws, bs, float(g["lr"]))
    assert loss == pytest.approx(float(g["loss"]), abs=5e-6)
    assert np.abs(logits - g["logits"]).max() < 2e-5
    for i in range(len(ws)):
        assert np.linalg.norm(grads[i][0]) == pytest.approx(float(g[f"dw{i}_norm"]), rel=1e-5)
        assert np.abs(new[i][0][:4, :16] - g[f"w{i}_new_head"]).max() < 1e-6
        assert np.abs(new[i][1] - g[f"b{i}_new"]).max() < 1e-6


def test_maxpool_routes_gradient_to_first_maximum(orc):
    x = np.zeros((1, 2, 2, 2), np.float16)
    x[0, :, :, 0] = [[1, 5], [5, 2]]     # tie between (0,1) and (1,0): first wins
    x[0, :, :, 1] = [[-1, -2], [-3, -0.5]]
    y, am = orc.maxpool2x2_fwd(x)
    assert y[0, 0, 0].tolist() == [5.0, -0.5] and am[0, 0, 0].tolist() == [1, 3]
    dx = orc.maxpool2x2_bwd(np.full((1, 1, 1, 2), 7, np.float16), am, x.shape)
    assert dx[0, 0, 1, 0] == 7 and dx[0, 1, 1, 1] == 7 and dx.astype(np.float32).sum() == 14


@pytest.mark.parametrize("k,stride,pad,h,w", [(3, 2, 1, 12, 9), (2, 2, 0, 8, 8), (3, 1, 1, 5, 7), (5, 3, 2, 11, 11)])
def test_general_pooling_restatements_against_torch(orc, k, stride, pad, h, w):
    """The numpy restatements of the reference's max pool (maxpool_op.cu:83-217) and global average pool
    (gap_op.cpp:137-155, gap_op.cu:92-112) against torch's operators and their autograd."""
    import torch
    import torch.nn.functional as F
    rng = np.random.default_rng(k * 10 + stride)
    n, c = 2, 8
    x = rng.standard_normal((n, h, w, c)).astype(np.float32)
    y, am = orc.maxpool_fwd(x, k, stride, pad)
    xt = torch.from_numpy(x).permute(0, 3, 1, 2).contiguous().requires_grad_(True)
    yt = F.max_pool2d(xt, k, stride, pad)
    assert np.array_equal(y, yt.detach().permute(0, 2, 3, 1).numpy())
    dy = rng.standard_normal(y.shape).astype(np.float32)
    yt.backward(torch.from_numpy(dy).permute(0, 3, 1, 2).contiguous())
    dx = orc.maxpool_bwd(dy, am, x.shape, k, stride, pad)
    assert np.allclose(dx, xt.grad.permute(0, 2, 3, 1).numpy(), rtol=1e-6, atol=1e-6)
    # argmax bytes decode to the position of the maximum inside the window
    kh, kw = am // k, am % k
    assert am.max() < k * k and (kh < k).all() and (kw < k).all()
    if (k, stride, pad) == (2, 2, 0):
        y2, am2 = orc.maxpool2x2_fwd(x.astype(np.float16))
        y16, am16 = orc.maxpool_fwd(x.astype(np.float16).astype(np.float32), 2, 2, 0)
        assert np.array_equal(y2.astype(np.float32), y16) and np.array_equal(am2, am16)
    g = orc.avgpool_global_fwd(x)
    assert np.allclose(g, x.mean(axis=(1, 2)), rtol=1e-5, atol=1e-6)
    dg = rng.standard_normal((n, c)).astype(np.float32)
    assert np.allclose(orc.avgpool_global_bwd(dg, h, w), np.broadcast_to(dg[:, None, None, :] / (h * w), x.shape),
                       rtol=1e-6)
