"""The CUDA kernels against vectors made by the reference project's own generator scripts
(tests/golden/ref_*.npz, see tests/golden/make_reference_golden.py).  The limits are the reference drivers'
(MSE <= 1e-3 for half tensors, tests/op/test_conv_fwd_bwd.cpp:366) together with BASELINE's relative ones."""
import numpy as np
import pytest
import torch

from conftest import golden, rel_l2, rel_max
from gpu_util import dev, host

pytestmark = pytest.mark.gpu


def mse(a, b):
    return float(np.mean((np.asarray(a, np.float64) - np.asarray(b, np.float64)) ** 2))


@pytest.mark.parametrize("name,tensor_cores", [("ref_conv_fp16_3x3_s1", False), ("ref_conv_fp16_3x3_s1_c64", True)])
def test_conv_forward_and_gradients_match_reference_generator(name, tensor_cores):
    from renaissance_b200 import ops
    g = golden(name)
    n, h, w, c, k, ker, stride, pad, _ = (int(v) for v in g["params"])
    geo = ops.ConvGeometry(n, h, w, c, k, ker, ker, pad, stride)
    assert ops.conv_uses_tensor_cores(geo, "dgrad") == tensor_cores
    assert ops.conv_uses_tensor_cores(geo, "wgrad") == tensor_cores
    x, wt, dy = dev(g["x_conv_amp"]), dev(g["w_conv_amp"]), dev(g["dy_conv_amp"])
    dw = ops.conv_wgrad(geo, dy, x)
    dx = ops.conv_dgrad(geo, dy, wt)
    ops.device_status()
    for got, ref in ((dw, g["dw_conv_ref_amp"]), (dx, g["dx_conv_ref_amp"])):
        got = host(got).astype(np.float32)
        assert mse(got, ref) <= 1e-3
        assert rel_l2(got, ref.astype(np.float32)) < 2e-2          # BASELINE's limit
        assert rel_l2(got, ref.astype(np.float32)) < 3e-3          # reached (the vectors themselves are half-rounded)
    if tensor_cores:
        y = ops.conv_fprop(geo, x, wt)
        ops.device_status()
        assert rel_l2(host(y).astype(np.float32), g["y_conv_ref_amp"].astype(np.float32)) < 3e-3
        _, st = ops.conv_fprop_bn_stats(geo, x, wt, torch.ones(k, device="cuda"), torch.zeros(k, device="cuda"),
                                        want_sums=True)
        ops.device_status()
        # the generator's per-channel sum and sum of squares of the (half-rounded) output
        assert rel_max(host(st["sum"]), g["sum_conv_ref_amp"].reshape(-1)) < 1e-3
        assert rel_max(host(st["sqsum"]), g["sq_sum_conv_ref_amp"].reshape(-1)) < 1e-3


def test_bn_backward_matches_reference_generator():
    """BN backward with no ReLU behind it (mask = NULL) on the generator's half case."""
    from renaissance_b200 import ops
    g = golden("ref_bn2d_fp16")
    v = lambda key: dev(g[f"{key}_amp"].reshape(-1))
    dx, dg, db = ops.bnrelu_bwd(dev(g["dy_bn_amp"]), None, dev(g["x_bn_amp"]), v("gamma_bn"), v("saved_mean_bn_ref"),
                                v("saved_inv_var_bn_ref"))
    assert rel_max(host(dg), g["dgamma_bn_ref_amp"].reshape(-1)) < 1e-4
    assert rel_max(host(db), g["dbeta_bn_ref_amp"].reshape(-1)) < 1e-4
    assert rel_l2(host(dx).astype(np.float32), g["dx_bn_ref_amp"].astype(np.float32)) < 2e-3


@pytest.mark.parametrize("name", ["ref_softmax_fp16_1000"])
def test_softmax_matches_reference_generator(name):
    from renaissance_b200 import ops
    g = golden(name)
    batch, classes, _ = (int(v) for v in g["params"])
    z = dev(g["logits_amp"].reshape(batch, classes))
    labels = dev(g["labels_fp32"].reshape(batch))
    sc = torch.tensor([1.0], device="cuda")
    ls = torch.tensor([0.0], device="cuda")
    ref_probs = g["softmax_probs_fp32"].reshape(batch, classes)
    ref_d = g["d_logits_amp"].reshape(batch, classes).astype(np.float32)
    ref_loss = float(g["ce_loss_fp32"].reshape(()))
    pred = g["pred_labels_fp32"].reshape(batch)
    # one fused pass
    out = ops.softmax_ce_amp_fused(z, labels, sc, ls, want_probs=True)
    assert abs(float(out["loss"]) - ref_loss) < 5e-5
    assert np.abs(host(out["probs"]) - ref_probs).max() < 5e-6
    assert np.array_equal(host(out["probs"]).argmax(axis=1).astype(np.int32), pred)      # bit-exact argmax
    assert mse(host(out["dlogits"]), ref_d) <= 1e-3 and rel_l2(host(out["dlogits"]).astype(np.float32), ref_d) < 1e-3
    # the two separate nodes
    f = ops.softmax_ce_amp_fwd(z, labels, ls)
    d = ops.softmax_ce_amp_bwd(f["probs"], labels, sc, f["inv_scaling"], ls)
    assert abs(float(f["loss"]) - ref_loss) < 5e-5
    assert np.abs(host(f["probs"]) - ref_probs).max() < 5e-6
    assert rel_l2(host(d).astype(np.float32), ref_d) < 1e-3
    # the lean fused kernel (probabilities not kept)
    lean = ops.softmax_ce_amp_fused(z, labels, sc, ls)
    assert abs(float(lean["loss"]) - ref_loss) < 5e-5
    assert rel_l2(host(lean["dlogits"]).astype(np.float32), ref_d) < 1e-3


@pytest.mark.parametrize("name", ["ref_maxpool_fp16_2x2_s2", "ref_maxpool_fp16_3x3_s2"])
def test_maxpool_matches_reference_generator(name):
    from renaissance_b200 import ops
    g = golden(name)
    n, h, w, c, k, stride, pad, _ = (int(v) for v in g["params"])
    x, dy = dev(g["x_fwd_bwd_amp"]), dev(g["dy_fwd_bwd_amp"])
    y, am = ops.maxpool_fwd(x, k, stride, pad)
    assert np.array_equal(host(y), g["y_ref_fwd_bwd_amp"])
    dx = ops.maxpool_bwd(dy, am, (n, h, w, c), k, stride, pad)
    if k == stride:
        assert np.array_equal(host(dx), g["dx_ref_fwd_bwd_amp"])
        y2, am2 = ops.maxpool2x2_fwd(x)
        assert np.array_equal(host(y2), g["y_ref_fwd_bwd_amp"])
        dx2 = ops.maxpool2x2_bwd(dy, am2, torch.empty_like(x))
        assert np.array_equal(host(dx2), g["dx_ref_fwd_bwd_amp"])
    else:
        assert rel_l2(host(dx).astype(np.float32), g["dx_ref_fwd_bwd_amp"].astype(np.float32)) < 1e-3
