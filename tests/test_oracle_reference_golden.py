"""Pins the CPU oracle to vectors made by the reference project's OWN generator scripts
(tests/golden/make_reference_golden.py imports tests/op/test_conv_fwd_bwd.py,
tests/op/test_bn_fwd_bwd_legacy.py, tests/correction/test_softmax_ce.py,
tests/op/test_maxpool_fwd_bwd.py and tests/correction/test_mlp_final.py from a checkout of the
reference and stores what they write).  Thresholds are the reference's own C++ drivers' (MSE
limits) plus the tighter figure the oracle actually reaches.  CPU only."""
import numpy as np
import pytest

from conftest import golden, rel_l2, rel_max

CONV = ["ref_conv_fp32_3x3_s1", "ref_conv_fp32_3x3_s2", "ref_conv_fp32_1x1_s1", "ref_conv_fp32_7x7_s2",
        "ref_conv_fp16_3x3_s1", "ref_conv_fp16_3x3_s1_c64"]


def mse(a, b):
    return float(np.mean((np.asarray(a, np.float64) - np.asarray(b, np.float64)) ** 2))


def test_every_fixture_names_the_reference_script_that_made_it():
    import glob
    import os
    from conftest import GOLDEN
    files = sorted(glob.glob(os.path.join(GOLDEN, "ref_*.npz")))
    assert len(files) >= 16
    for f in files:
        prov = str(np.load(f)["provenance"])
        assert prov.startswith(("tests/op/test_", "tests/correction/test_")) and "::generate" in prov


@pytest.mark.parametrize("name", CONV)
def test_conv_matches_reference_generator(orc, name):
    g = golden(name)
    n, h, w, c, k, ker, stride, pad, half = (int(v) for v in g["params"])
    sfx = "_amp" if half else "_fp32"
    x, wt, dy = (g[f"{t}_conv{sfx}"].astype(np.float32) for t in ("x", "w", "dy"))
    y = orc.conv_fwd(x, wt, pad=pad, stride=stride)
    dx = orc.conv_dgrad(dy, wt, x.shape, pad=pad, stride=stride)
    dw = orc.conv_wgrad(dy, x, wt.shape, pad=pad, stride=stride)
    # reference thresholds: MSE <= 1e-5 in float, <= 1e-3 in half (the generator's mse_threshold)
    lim, tight = (1e-3, 2e-3) if half else (1e-5, 3e-6)
    for got, ref in ((y, g[f"y_conv_ref{sfx}"]), (dx, g[f"dx_conv_ref{sfx}"]), (dw, g[f"dw_conv_ref{sfx}"])):
        assert got.shape == ref.shape
        assert mse(got, ref) <= lim
        assert rel_l2(got, ref.astype(np.float32)) < tight     # half cases: the stored vectors are half-rounded
    if not half:
        assert rel_max(y.sum(axis=(0, 1, 2)), g[f"sum_conv_ref{sfx}"]) < 1e-5
        assert rel_max((y ** 2).sum(axis=(0, 1, 2)), g[f"sq_sum_conv_ref{sfx}"]) < 1e-5


@pytest.mark.parametrize("name", ["ref_bn2d_fp32", "ref_bn1d_fp32", "ref_bn2d_fp16"])
def test_bn_matches_reference_generator(orc, name):
    g = golden(name)
    half = name.endswith("fp16")
    sfx = "_amp" if half else "_fp32"
    c = int(g["params"][3])
    v = lambda key: g[f"{key}{sfx}"].reshape(-1)
    x = g[f"x_bn{sfx}"].astype(np.float32)
    rm, rv = v("running_mean_init_bn").copy(), v("running_var_init_bn").copy()
    y, mean, inv = orc.bn_fwd(x, v("gamma_bn"), v("beta_bn"), rm, rv, float(v("eps_bn")[0]), float(v("momentum_bn")[0]))
    assert np.allclose(mean, v("saved_mean_bn_ref"), atol=1e-6)
    assert rel_max(inv, v("saved_inv_var_bn_ref")) < 1e-6
    assert np.allclose(rm, v("running_mean_new_bn"), atol=1e-6)
    assert rel_max(rv, v("running_var_new_bn")) < 1e-6
    dx, dg, db = orc.bn_bwd(g[f"dy_bn{sfx}"].astype(np.float32), x, v("gamma_bn"), mean, inv)
    tol = 1e-3 if half else 1e-5            # the half case stores y and dx rounded to half
    assert rel_l2(y, g[f"y_bn_ref{sfx}"].astype(np.float32)) < tol
    assert rel_l2(dx, g[f"dx_bn_ref{sfx}"].astype(np.float32)) < tol
    assert rel_max(dg, v("dgamma_bn_ref")) < 1e-5
    assert rel_max(db, v("dbeta_bn_ref")) < 1e-5
    assert dg.shape == (c,)


@pytest.mark.parametrize("name", ["ref_softmax_fp32_1000", "ref_softmax_fp16_1000", "ref_softmax_fp32_10"])
def test_softmax_cpu_operator_matches_reference_generator(orc, name):
    g = golden(name)
    batch, classes, _ = (int(v) for v in g["params"])
    z = g["logits_fp32"].reshape(batch, classes).astype(np.float32)
    labels = g["labels_fp32"].reshape(batch)
    loss, inv, probs = orc.softmax_ce_fwd_cpu(z, labels, scaling=1.0, ls=0.0)
    # reference thresholds: loss / probs / d_logits MSE <= 1e-6 (tests/correction/test_softmax_ce.cpp:319-353)
    assert abs(loss - float(g["ce_loss_fp32"].reshape(()))) < 2e-5
    assert inv == pytest.approx(1.0 / batch)
    assert np.abs(probs - g["softmax_probs_fp32"].reshape(batch, classes)).max() < 1e-6
    d = orc.softmax_ce_bwd(probs, labels, scale=1.0 * inv, ls=0.0)
    assert np.abs(d - g["d_logits_fp32"].reshape(batch, classes)).max() < 1e-6
    assert np.array_equal(probs.argmax(axis=1).astype(np.int32), g["pred_labels_fp32"].reshape(batch))
    top1 = float((probs.argmax(axis=1) == labels).mean())
    assert top1 == pytest.approx(float(g["top1_correct_fp32"].reshape(())))


def test_softmax_amp_operator_matches_reference_generator(orc):
    """The AMP operator (half logits in, float probabilities, half gradient; softmax_ce_op.cu:63-177, 438-468)
    against the generator's fp16 case."""
    g = golden("ref_softmax_fp16_1000")
    batch, classes, _ = (int(v) for v in g["params"])
    z16 = g["logits_amp"].reshape(batch, classes)
    assert z16.dtype == np.float16
    labels = g["labels_fp32"].reshape(batch)
    out = orc.softmax_ce_amp(z16, labels, scaling=1.0, ls=0.0)
    assert abs(out["loss"] - float(g["ce_loss_fp32"].reshape(()))) < 5e-5
    assert np.abs(out["probs"] - g["softmax_probs_fp32"].reshape(batch, classes)).max() < 1e-6
    ref = g["d_logits_amp"].reshape(batch, classes).astype(np.float32)
    assert mse(out["dlogits"], ref) <= 1e-3 and rel_l2(out["dlogits"].astype(np.float32), ref) < 1e-3
    assert np.array_equal(out["probs"].argmax(axis=1).astype(np.int32), g["pred_labels_fp32"].reshape(batch))


@pytest.mark.parametrize("name", ["ref_maxpool_fp16_2x2_s2", "ref_maxpool_fp16_3x3_s2", "ref_maxpool_fp32_2x2_s2"])
def test_maxpool_matches_reference_generator(orc, name):
    g = golden(name)
    n, h, w, c, k, stride, pad, half = (int(v) for v in g["params"])
    sfx = "_amp" if half else "_fp32"
    x, dy = g[f"x_fwd_bwd{sfx}"], g[f"dy_fwd_bwd{sfx}"]
    y, am = orc.maxpool_fwd(x, k, stride, pad)
    assert np.array_equal(y.astype(x.dtype), g[f"y_ref_fwd_bwd{sfx}"])            # a selection: bit-exact
    dx = orc.maxpool_bwd(dy, am, x.shape, k, stride, pad)
    ref = g[f"dx_ref_fwd_bwd{sfx}"].astype(np.float32)
    if k == stride:                                                            # no overlap: a scatter, bit-exact
        assert np.array_equal(dx.astype(x.dtype), g[f"dx_ref_fwd_bwd{sfx}"])
    else:                                                                      # overlapping windows add in float
        assert rel_l2(dx, ref) < 1e-3
    if half and k == 2:
        y2, am2 = orc.maxpool2x2_fwd(x)
        assert np.array_equal(y2, g[f"y_ref_fwd_bwd{sfx}"])
        assert np.array_equal(orc.maxpool2x2_bwd(dy, am2, x.shape), g[f"dx_ref_fwd_bwd{sfx}"])


def test_fc_and_softmax_match_reference_mlp_generator(orc):
    """tests/correction/test_mlp_final.py is Flatten-FC-Tanh-FC-Tanh-FC-SoftmaxCE; every FC forward / backward and the
    loss head are checked in isolation on the tensors the generator stored either side of them (Tanh is not on this
    library's path).  The reference's threshold is MSE <= 1e-5 in float."""
    g = golden("ref_mlp_final_fp32")
    t = lambda key: g[f"{key}_fp32"]
    m = lambda key: t(key).reshape(t(key).shape[0], -1) if t(key).shape[0] != 1 else t(key).reshape(-1)
    batch = 7
    # forward
    y1 = orc.fc_fwd(m("flat_out"), m("w1"), m("b1")[:32])
    assert rel_l2(y1, m("fc1_out")[:, :32]) < 1e-5
    y2 = orc.fc_fwd(m("tanh1_out"), m("w2"), m("b2"))
    assert rel_l2(y2, m("fc2_out")) < 1e-5
    y3 = orc.fc_fwd(m("tanh2_out"), m("w3"), m("b3"))
    assert rel_l2(y3, m("logits")) < 1e-5
    # loss head
    labels = t("labels").reshape(batch)
    loss, inv, probs = orc.softmax_ce_fwd_cpu(m("logits"), labels, scaling=1.0, ls=0.0)
    assert abs(loss - float(t("loss").reshape(()))) < 2e-5
    assert inv == pytest.approx(float(t("inv_scaling").reshape(())))
    assert np.abs(probs - m("probs")).max() < 1e-6
    d = orc.softmax_ce_bwd(probs, labels, scale=inv, ls=0.0)
    assert np.abs(d - m("d_logits")).max() < 1e-6
    # backward
    dx3, dw3, db3 = orc.fc_bwd(m("d_logits"), m("w3"), m("tanh2_out"))
    assert rel_l2(dx3, m("d_tanh2_ref")) < 1e-5 and rel_l2(dw3, m("dw3_ref")) < 1e-5 and rel_l2(db3, m("db3_ref")) < 1e-5
    dx2, dw2, db2 = orc.fc_bwd(m("d_fc2_ref"), m("w2"), m("tanh1_out"))
    assert rel_l2(dx2, m("d_tanh1_ref")) < 1e-5 and rel_l2(db2, m("db2_ref")) < 1e-5
    assert rel_l2(dw2[:32], m("dw2_ref")) < 1e-5
    _, dw1, db1 = orc.fc_bwd(m("d_fc1_ref")[:, :32], m("w1"), m("flat_out"))
    assert rel_l2(dw1, m("dw1_ref")) < 1e-5 and rel_l2(db1, m("db1_ref")[:32]) < 1e-5
    assert mse(dw1, m("dw1_ref")) <= 1e-5
