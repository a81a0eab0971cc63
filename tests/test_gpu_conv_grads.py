"""Convolution weight / data gradients: direct kernels (any geometry) and the
tcgen05 implicit-GEMM kernels (3x3 s1 p1, channels % 64 == 0) against the oracle."""
import numpy as np
import pytest
import torch

from conftest import golden, rel_l2
from gpu_util import dev, host

pytestmark = pytest.mark.gpu


def _rand_case(seed, n, h, w, c, k, r, pad, stride):
    rng = np.random.default_rng(seed)
    oh = (h + 2 * pad - r) // stride + 1
    ow = (w + 2 * pad - r) // stride + 1
    x = rng.standard_normal((n, h, w, c)).astype(np.float16)
    wt = (rng.standard_normal((k, r, r, c)) * np.sqrt(2.0 / (r * r * c))).astype(np.float16)
    dy = rng.standard_normal((n, oh, ow, k)).astype(np.float16)
    return x, wt, dy


def _oracle(orc, x, wt, dy, pad, stride):
    dw = orc.conv_wgrad(dy.astype(np.float32), x.astype(np.float32), wt.shape, pad=pad, stride=stride)
    dx = orc.conv_dgrad(dy.astype(np.float32), wt.astype(np.float32), x.shape, pad=pad, stride=stride)
    return dw, dx


DIRECT_CASES = [
    (1, 5, 5, 3, 8, 3, 1, 1), (2, 9, 7, 4, 8, 3, 1, 2), (1, 12, 12, 3, 8, 7, 3, 2), (2, 8, 8, 16, 24, 1, 0, 1),
    (3, 6, 10, 8, 8, 5, 2, 1), (2, 16, 16, 4, 24, 3, 1, 1),
]


@pytest.mark.parametrize("n,h,w,c,k,r,pad,stride", DIRECT_CASES)
def test_direct_kernels_match_oracle(orc, n, h, w, c, k, r, pad, stride):
    from renaissance_b200 import ops
    x, wt, dy = _rand_case(n * 7 + h, n, h, w, c, k, r, pad, stride)
    ref_dw, ref_dx = _oracle(orc, x, wt, dy, pad, stride)
    g = ops.ConvGeometry(n, h, w, c, k, r, r, pad, stride)
    assert not ops.conv_uses_tensor_cores(g, "wgrad")
    dw = ops.conv_wgrad(g, dev(dy), dev(x))
    dx = ops.conv_dgrad(g, dev(dy), dev(wt))
    torch.cuda.synchronize()
    assert rel_l2(host(dw).astype(np.float32), ref_dw) < 2e-2
    assert rel_l2(host(dx).astype(np.float32), ref_dx) < 2e-2
    assert rel_l2(host(dw).astype(np.float32), ref_dw) < 2e-3 and rel_l2(host(dx).astype(np.float32), ref_dx) < 2e-3


def test_direct_kernels_match_golden():
    from renaissance_b200 import ops
    g = golden("conv_fp16_3x3_s1")
    n, h, w, c, k, ker, stride, pad, _ = (int(v) for v in g["params"])
    geo = ops.ConvGeometry(n, h, w, c, k, ker, ker, pad, stride)
    dw = ops.conv_wgrad(geo, dev(g["dy"], torch.float16), dev(g["x"], torch.float16))
    dx = ops.conv_dgrad(geo, dev(g["dy"], torch.float16), dev(g["w"], torch.float16))
    # the reference's AMP threshold is MSE <= 1e-3 (tests/op/test_conv_fwd_bwd.cpp:366)
    assert rel_l2(host(dw).astype(np.float32), g["dw"]) < 2e-3
    assert rel_l2(host(dx).astype(np.float32), g["dx"]) < 2e-3


IGEMM_CASES = [
    # n, h, w, c, k        what it exercises
    (2, 8, 8, 64, 64),      # one tile, N tile 64
    (1, 16, 8, 64, 128),    # N tile 128
    (3, 7, 5, 64, 64),      # odd extents: boxes hang over every edge
    (2, 14, 14, 128, 256),  # 14x14: tile 2x2x32 images, N tile 256, two input slices
    (5, 12, 20, 256, 64),   # four input slices, several tiles
    (2, 28, 28, 128, 128),
    (1, 9, 33, 64, 512),    # two N tiles
    (4, 14, 14, 512, 512),  # deep VGG shape at a small batch
    (2, 11, 13, 128, 64),   # channels-as-M tile of 64 over two input slices, ragged last pixel tile
    (1, 6, 6, 256, 128),    # four input slices, fewer pixels than one 256-pixel tile
    (5, 3, 3, 64, 128),     # images smaller than the filter's reach on every side
    (2, 17, 9, 256, 64),    # wgrad units spread over more split-K parts than pixel tiles
]


@pytest.mark.parametrize("n,h,w,k", [(2, 16, 16, 64), (3, 9, 7, 128), (2, 20, 12, 256), (2, 32, 64, 64),
                                     (5, 6, 2, 64), (1, 40, 130, 64), (70, 1, 2, 64)])
def test_first_layer_four_channels_on_tensor_cores(orc, n, h, w, k):
    """c = 4 (3 image channels + 1 pad): forward and weight gradient as a 1x1 GEMM over
    the pixels' 3x3 neighbourhoods, which the kernels build in shared memory (from halo tiles
    fetched by TMA, or with plain loads when the width is odd or the halo tile is too large)."""
    from renaissance_b200 import ops
    x, wt, dy = _rand_case(n * 5 + k, n, h, w, 4, k, 3, 1, 1)
    x[..., 3] = 0
    ref_dw, _ = _oracle(orc, x, wt, dy, 1, 1)
    g = ops.ConvGeometry(n, h, w, 4, k)
    assert ops.conv_uses_tensor_cores(g, "wgrad") and ops.conv_uses_tensor_cores(g, "fprop")
    assert not ops.conv_uses_tensor_cores(g, "dgrad")
    dw = ops.conv_wgrad(g, dev(dy), dev(x))
    y = ops.conv_fprop(g, dev(x), dev(wt))
    ops.device_status()
    assert rel_l2(host(dw).astype(np.float32), ref_dw) < 2e-3
    assert rel_l2(host(y).astype(np.float32), orc.conv_fwd(x.astype(np.float32), wt.astype(np.float32))) < 2e-3
    ops.set_conv_backend(direct_only=True)
    try:
        dw_direct = ops.conv_wgrad(g, dev(dy), dev(x))
    finally:
        ops.set_conv_backend(direct_only=False)
    assert rel_l2(host(dw).astype(np.float32), host(dw_direct).astype(np.float32)) < 2e-3


@pytest.mark.parametrize("n,h,w,c,k", IGEMM_CASES)
def test_tensor_core_kernels_match_oracle(orc, n, h, w, c, k):
    from renaissance_b200 import ops
    x, wt, dy = _rand_case(n + h * 3 + c, n, h, w, c, k, 3, 1, 1)
    ref_dw, ref_dx = _oracle(orc, x, wt, dy, 1, 1)
    g = ops.ConvGeometry(n, h, w, c, k)
    assert ops.conv_uses_tensor_cores(g, "wgrad") and ops.conv_uses_tensor_cores(g, "dgrad")
    dw = ops.conv_wgrad(g, dev(dy), dev(x))
    dx = ops.conv_dgrad(g, dev(dy), dev(wt))
    y = ops.conv_fprop(g, dev(x), dev(wt))
    ops.device_status()
    ref_y = orc.conv_fwd(x.astype(np.float32), wt.astype(np.float32))
    assert rel_l2(host(dx).astype(np.float32), ref_dx) < 2e-3
    assert rel_l2(host(dw).astype(np.float32), ref_dw) < 2e-3
    assert rel_l2(host(y).astype(np.float32), ref_y) < 2e-3


@pytest.mark.parametrize("n,h,w,c,k", [(2, 8, 8, 64, 64), (3, 7, 5, 128, 256), (2, 14, 14, 256, 64),
                                       (1, 9, 33, 512, 128), (4, 7, 7, 1024, 512), (2, 28, 28, 64, 256)])
def test_one_by_one_convolutions_on_tensor_cores(orc, n, h, w, c, k):
    """1x1 stride 1: the same kernels with one filter tap (a plain GEMM over the pixels)."""
    from renaissance_b200 import ops
    x, wt, dy = _rand_case(n + h + c + k, n, h, w, c, k, 1, 0, 1)
    ref_dw, ref_dx = _oracle(orc, x, wt, dy, 0, 1)
    g = ops.ConvGeometry(n, h, w, c, k, 1, 1, 0, 1)
    for which in ("wgrad", "dgrad", "fprop"):
        assert ops.conv_uses_tensor_cores(g, which)
    dw = ops.conv_wgrad(g, dev(dy), dev(x))
    dx = ops.conv_dgrad(g, dev(dy), dev(wt))
    y = ops.conv_fprop(g, dev(x), dev(wt))
    gamma, beta = np.ones(k, np.float32), np.zeros(k, np.float32)
    y2, st = ops.conv_fprop_bn_stats(g, dev(x), dev(wt), dev(gamma), dev(beta), want_sums=True)
    ops.device_status()
    assert rel_l2(host(dx).astype(np.float32), ref_dx) < 2e-3
    assert rel_l2(host(dw).astype(np.float32), ref_dw) < 2e-3
    assert rel_l2(host(y).astype(np.float32), orc.conv_fwd(x.astype(np.float32), wt.astype(np.float32), pad=0)) < 2e-3
    assert torch.equal(y, y2)
    yf = host(y).astype(np.float64).reshape(-1, k)
    assert rel_l2(host(st["sum"]), yf.sum(axis=0)) < 1e-4
    ops.set_conv_backend(direct_only=True)
    try:
        dw3, dx3 = ops.conv_wgrad(g, dev(dy), dev(x)), ops.conv_dgrad(g, dev(dy), dev(wt))
    finally:
        ops.set_conv_backend(direct_only=False)
    assert rel_l2(host(dw).astype(np.float32), host(dw3).astype(np.float32)) < 2e-3
    assert rel_l2(host(dx).astype(np.float32), host(dx3).astype(np.float32)) < 2e-3


@pytest.mark.parametrize("n,h,w,c,k,r,pad", [(2, 8, 8, 64, 64, 3, 1), (2, 9, 7, 64, 128, 3, 1), (1, 14, 14, 128, 256, 3, 1),
                                             (3, 8, 8, 128, 64, 1, 0), (2, 7, 9, 256, 512, 1, 0),
                                             (2, 28, 28, 64, 128, 1, 0)])
def test_stride_two_convolutions_on_tensor_cores(orc, n, h, w, c, k, r, pad):
    """Stride 2 (3x3 pad 1, 1x1 pad 0) on the tensor-core kernels (stepped tensor maps, parity classes of the data
    gradient), against the oracle's strided loops and the direct strided kernels; odd extents included.  The forward
    with the statistics epilogue gives the same output and the sums of that output."""
    from renaissance_b200 import ops
    x, wt, dy = _rand_case(n + h + c + k + r, n, h, w, c, k, r, pad, 2)
    ref_dw, ref_dx = _oracle(orc, x, wt, dy, pad, 2)
    g = ops.ConvGeometry(n, h, w, c, k, r, r, pad, 2)
    for which in ("wgrad", "dgrad", "fprop"):
        assert ops.conv_uses_tensor_cores(g, which)
    dw = ops.conv_wgrad(g, dev(dy), dev(x))
    dx = ops.conv_dgrad(g, dev(dy), dev(wt))
    y = ops.conv_fprop(g, dev(x), dev(wt))
    ops.device_status()
    assert tuple(y.shape) == tuple(dy.shape)
    assert rel_l2(host(dx).astype(np.float32), ref_dx) < 2e-3
    assert rel_l2(host(dw).astype(np.float32), ref_dw) < 2e-3
    ref_y = orc.conv_fwd(x.astype(np.float32), wt.astype(np.float32), pad=pad, stride=2)
    assert rel_l2(host(y).astype(np.float32), ref_y) < 2e-3
    gamma, beta = torch.ones(k, device="cuda"), torch.zeros(k, device="cuda")
    y2, st = ops.conv_fprop_bn_stats(g, dev(x), dev(wt), gamma, beta, want_sums=True)
    assert torch.equal(y2, y)
    rows = y.double().reshape(-1, k)
    assert float((st["sum"].double() - rows.sum(dim=0)).abs().max() / rows.abs().sum(dim=0).max()) < 1e-5
    assert float((st["sqsum"].double() - (rows * rows).sum(dim=0)).abs().max() / (rows * rows).sum(dim=0).max()) < 1e-5
    ops.set_conv_backend(direct_only=True)
    try:
        dw3, dx3 = ops.conv_wgrad(g, dev(dy), dev(x)), ops.conv_dgrad(g, dev(dy), dev(wt))
    finally:
        ops.set_conv_backend(direct_only=False)
    assert rel_l2(host(dw).astype(np.float32), host(dw3).astype(np.float32)) < 2e-3
    assert rel_l2(host(dx).astype(np.float32), host(dx3).astype(np.float32)) < 2e-3


@pytest.mark.parametrize("n,h,w,k,r,pad,stride,dtype", [
    (2, 32, 32, 64, 7, 3, 2, torch.float16), (1, 17, 23, 128, 5, 2, 1, torch.float16),
    (3, 20, 12, 64, 7, 3, 2, torch.bfloat16), (2, 16, 16, 64, 3, 1, 1, torch.bfloat16),
    (2, 15, 15, 256, 3, 0, 2, torch.float16)])
def test_first_layers_lowered_to_rows(orc, n, h, w, k, r, pad, stride, dtype):
    """Four input channels with any filter, stride and padding: receptive fields written out as rows, then a
    1x1 convolution on the tensor cores (forward and weight gradient)."""
    from renaissance_b200 import ops
    x, wt, dy = _rand_case(n + h + k + r, n, h, w, 4, k, r, pad, stride)
    x[..., 3] = 0
    if dtype == torch.bfloat16:
        rnd = lambda a: torch.from_numpy(a.astype(np.float32)).bfloat16().float().numpy()   # noqa: E731
        x, wt, dy = rnd(x), rnd(wt), rnd(dy)
    x32, w32, dy32 = (a.astype(np.float32) for a in (x, wt, dy))
    g = ops.ConvGeometry(n, h, w, 4, k, r, r, pad, stride, dtype=dtype)
    assert ops.conv_uses_tensor_cores(g, "wgrad") and ops.conv_uses_tensor_cores(g, "fprop")
    assert not ops.conv_uses_tensor_cores(g, "dgrad")
    dw = ops.conv_wgrad(g, dev(dy32).to(dtype), dev(x32).to(dtype))
    y = ops.conv_fprop(g, dev(x32).to(dtype), dev(w32).to(dtype))
    ops.device_status()
    tol = 2e-3 if dtype == torch.float16 else 4e-3
    assert rel_l2(host(dw.float()), orc.conv_wgrad(dy32, x32, wt.shape, pad=pad, stride=stride)) < tol
    assert rel_l2(host(y.float()), orc.conv_fwd(x32, w32, pad=pad, stride=stride)) < tol


def test_tensor_core_kernels_are_bitwise_reproducible_and_agree_with_direct():
    from renaissance_b200 import ops
    n, h, w, c, k = 8, 28, 28, 128, 256
    x, wt, dy = _rand_case(99, n, h, w, c, k, 3, 1, 1)
    g = ops.ConvGeometry(n, h, w, c, k)
    xd, wd, dyd = dev(x), dev(wt), dev(dy)
    dw1, dx1 = ops.conv_wgrad(g, dyd, xd), ops.conv_dgrad(g, dyd, wd)
    dw2, dx2 = ops.conv_wgrad(g, dyd, xd), ops.conv_dgrad(g, dyd, wd)
    ops.device_status()
    assert torch.equal(dw1, dw2) and torch.equal(dx1, dx2)
    ops.set_conv_backend(direct_only=True)
    try:
        dw3, dx3 = ops.conv_wgrad(g, dyd, xd), ops.conv_dgrad(g, dyd, wd)
    finally:
        ops.set_conv_backend(direct_only=False)
    torch.cuda.synchronize()
    assert rel_l2(host(dw1).astype(np.float32), host(dw3).astype(np.float32)) < 2e-3
    assert rel_l2(host(dx1).astype(np.float32), host(dx3).astype(np.float32)) < 2e-3


def test_full_size_config2_against_torch_fp32():
    """BASELINE.json configuration 2 (N=256, 56x56, C=K=64): too large for the CPU oracle in a
    test, so the check is against torch's float32 convolution gradients on the GPU
    plus linearity in dy."""
    from renaissance_b200 import ops
    n, h, w, c, k = 256, 56, 56, 64, 64
    gen = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn((n, h, w, c), generator=gen, device="cuda").half()
    wt = (torch.randn((k, 3, 3, c), generator=gen, device="cuda") * (2.0 / (9 * c)) ** 0.5).half()
    dy = torch.randn((n, h, w, k), generator=gen, device="cuda").half()
    g = ops.ConvGeometry(n, h, w, c, k)
    dw = ops.conv_wgrad(g, dy, x)
    dx = ops.conv_dgrad(g, dy, wt)
    dx_half = ops.conv_dgrad(g, (dy.float() * 0.5).half(), wt)
    ops.device_status()
    assert float((dx_half.float() * 2 - dx.float()).abs().max()) <= 2e-3 * float(dx.float().abs().max())
    torch.backends.cudnn.allow_tf32 = False
    xn = x.float().permute(0, 3, 1, 2).contiguous().requires_grad_(True)
    wn = wt.float().permute(0, 3, 1, 2).contiguous().requires_grad_(True)
    out = torch.nn.functional.conv2d(xn, wn, padding=1)
    out.backward(dy.float().permute(0, 3, 1, 2).contiguous())
    ref_dx = xn.grad.permute(0, 2, 3, 1)
    ref_dw = wn.grad.permute(0, 2, 3, 1)
    assert float((dx.float() - ref_dx).norm() / ref_dx.norm()) < 2e-3
    assert float((dw.float() - ref_dw).norm() / ref_dw.norm()) < 2e-3
