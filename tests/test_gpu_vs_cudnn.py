"""This repository's kernels against the reference's cuDNN path on identical seeded inputs.

The reference executes its block through cuDNN-frontend graphs (cbr_op.cpp:430-917, 1259-1353);
cudnn_reference.py (beside bench.py) rebuilds those graphs with the cudnn-frontend Python package.  Tolerances are
BASELINE.json's: <= 2e-2 relative L2 for half dx / dW (both sides round to half, ~1e-3 is what is reached), <= 1e-4
relative for the per-channel reductions against a float64 evaluation (cuDNN's own reduction order differs)."""
import numpy as np
import pytest
import torch

from gpu_util import dev, host  # noqa: F401
from conftest import rel_l2

pytestmark = pytest.mark.gpu


def _cr():
    import cudnn_reference as cr
    if not cr.available():
        pytest.skip("cudnn-frontend Python package not present")
    return cr


@pytest.mark.parametrize("n,h,w,c,k", [(8, 28, 28, 64, 64), (4, 14, 14, 128, 256), (2, 56, 56, 64, 128),
                                       (3, 9, 11, 256, 64)])
def test_conv_kernels_match_cudnn_graphs(n, h, w, c, k):
    from renaissance_b200 import ops
    cr = _cr()
    g = torch.Generator(device="cuda").manual_seed(n * 7 + c)
    x = torch.randn((n, h, w, c), generator=g, device="cuda").half()
    wt = (torch.randn((k, 3, 3, c), generator=g, device="cuda") * (2.0 / (9 * c)) ** 0.5).half()
    dy = torch.randn((n, h, w, k), generator=g, device="cuda").half()
    geo = ops.ConvGeometry(n, h, w, c, k)
    ours = dict(y=ops.conv_fprop(geo, x, wt), dx=ops.conv_dgrad(geo, dy, wt), dw=ops.conv_wgrad(geo, dy, x))
    ops.device_status()
    ref = dict(y=torch.empty_like(dy), dx=torch.empty_like(x), dw=torch.empty_like(wt))
    cr.conv_fprop(x, wt, ref["y"])()
    cr.conv_dgrad(dy, wt, ref["dx"])()
    cr.conv_wgrad(x, dy, ref["dw"])()
    torch.cuda.synchronize()
    for name in ("y", "dx", "dw"):
        assert rel_l2(host(ours[name]).astype(np.float32), host(ref[name]).astype(np.float32)) < 2e-3, name


@pytest.mark.parametrize("r,c,k,h,stride,pad", [(1, 64, 256, 28, 1, 0), (1, 512, 128, 14, 1, 0), (3, 128, 128, 28, 1, 1),
                                                (3, 128, 128, 28, 2, 1), (1, 256, 512, 28, 2, 0), (1, 2048, 512, 7, 1, 0)])
def test_resnet50_shapes_bf16_match_cudnn_graphs(r, c, k, h, stride, pad):
    """bfloat16 gradients of ResNet-50 convolution shapes (1x1, 3x3, strided) against cuDNN's graphs."""
    from renaissance_b200 import ops
    cr = _cr()
    n = 4
    g = torch.Generator(device="cuda").manual_seed(r + c + k)
    geo = ops.ConvGeometry(n, h, h, c, k, r, r, pad, stride, dtype=torch.bfloat16)
    x = torch.randn((n, h, h, c), generator=g, device="cuda").bfloat16()
    wt = (torch.randn((k, r, r, c), generator=g, device="cuda") * (2.0 / (r * r * c)) ** 0.5).bfloat16()
    dy = torch.randn((n, geo.oh, geo.ow, k), generator=g, device="cuda").bfloat16()
    ours = dict(dx=ops.conv_dgrad(geo, dy, wt), dw=ops.conv_wgrad(geo, dy, x))
    ops.device_status()
    ref = dict(dx=torch.empty_like(x), dw=torch.empty_like(wt))
    cr.conv_dgrad(dy, wt, ref["dx"], pad=pad, stride=stride)()
    cr.conv_wgrad(x, dy, ref["dw"], pad=pad, stride=stride)()
    torch.cuda.synchronize()
    for name in ("dx", "dw"):
        # both sides round to bfloat16 (8 significant bits): 2e-2 is the stated bound, ~3e-3 what is reached
        err = rel_l2(host(ours[name].float()), host(ref[name].float()))
        assert err < 2e-2 and err < 6e-3, (name, err)


def test_conv_statistics_match_cudnn_genstats():
    from renaissance_b200 import ops
    cr = _cr()
    n, h, w, c, k = 8, 28, 28, 64, 128
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn((n, h, w, c), generator=g, device="cuda").half()
    wt = (torch.randn((k, 3, 3, c), generator=g, device="cuda") * (2.0 / (9 * c)) ** 0.5).half()
    gamma, beta = torch.ones(k, device="cuda"), torch.zeros(k, device="cuda")
    _, out = ops.conv_fprop_bn_stats(ops.ConvGeometry(n, h, w, c, k), x, wt, gamma, beta)
    ops.device_status()
    y = torch.empty((n, h, w, k), device="cuda", dtype=torch.float16)
    s, q = torch.empty(k, device="cuda"), torch.empty(k, device="cuda")
    try:
        cr.conv_fprop(x, wt, y, genstats=(s, q))()
    except Exception:
        # this cuDNN build has no engine for conv + genstats on this GPU: take the sums of the cuDNN conv output
        cr.conv_fprop(x, wt, y)()
        yf = y.float().reshape(-1, k)
        s, q = yf.sum(dim=0), (yf * yf).sum(dim=0)
    torch.cuda.synchronize()
    m = n * h * w
    mean_ref = (s / m).double()
    var_ref = (q / m).double() - mean_ref ** 2
    assert rel_l2(host(out["saved_mean"]).astype(np.float64), host(mean_ref)) < 1e-3
    inv_ref = 1.0 / torch.sqrt(var_ref + 1e-5)
    assert rel_l2(host(out["saved_inv_std"]).astype(np.float64), host(inv_ref)) < 1e-3


@pytest.mark.parametrize("n,h,w,c", [(8, 28, 28, 64), (4, 14, 14, 256), (2, 9, 7, 128)])
def test_bnrelu_backward_matches_cudnn_graph(n, h, w, c):
    from renaissance_b200 import ops
    cr = _cr()
    m = n * h * w
    g = torch.Generator(device="cuda").manual_seed(c + m)
    dy = torch.randn((m, c), generator=g, device="cuda").half()
    x = (torch.randn((m, c), generator=g, device="cuda") * 1.5 + 0.3).half()
    bits = torch.randint(0, 256, (m * c // 8,), generator=g, device="cuda", dtype=torch.int32).to(torch.uint8)
    gamma = 1 + 0.2 * torch.randn(c, generator=g, device="cuda")
    mean = x.float().mean(dim=0)
    inv = 1.0 / torch.sqrt(x.float().var(dim=0, unbiased=False) + 1e-5)
    o_dconv, o_dgamma, o_dbeta = ops.bnrelu_bwd(dy, bits, x, gamma, mean, inv)
    ops.device_status()
    dx, dg, db = torch.empty_like(dy), torch.empty(c, device="cuda"), torch.empty(c, device="cuda")
    cr.bnrelu_bwd(dy, bits, x, gamma, mean, inv, dx, dg, db, nhw=(n, h, w))()
    torch.cuda.synchronize()
    assert rel_l2(host(o_dconv).astype(np.float32), host(dx).astype(np.float32)) < 2e-3
    assert rel_l2(host(o_dgamma), host(dg)) < 1e-4
    assert rel_l2(host(o_dbeta), host(db)) < 1e-4
