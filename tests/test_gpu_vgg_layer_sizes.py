"""Parity at the sizes the VGG16-BN benchmark itself runs (batch 256): tensors of 1.6 GB whose byte offsets pass
2^31, where index arithmetic that wraps would hide from the small cases.  Too large for the CPU oracle, so the
reference is torch in float32 (float64 for the reductions) on the GPU, computed image by image; convolutions are
compared on images from the start, the middle and the end of the batch (each image is an independent problem for
forward and data gradient) and the weight gradient, a sum over the whole batch, on all of it in chunks.
Tolerances: BASELINE's 2e-2 relative L2 for half tensors (2e-3 asserted), 1e-4 relative for channel reductions,
bit-exact masks and argmax."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

N = 256
IMAGES = (0, 1, 127, 254, 255)


def _nchw(t):
    return t.float().permute(0, 3, 1, 2).contiguous()


def _nhwc(t):
    return t.permute(0, 2, 3, 1).contiguous()


def _rel(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm())


def _tensors(h, c, k, seed):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn((N, h, h, c), generator=gen, device="cuda").half()
    wt = (torch.randn((k, 3, 3, c), generator=gen, device="cuda") * (2.0 / (9 * c)) ** 0.5).half()
    dy = torch.randn((N, h, h, k), generator=gen, device="cuda").half()
    return x, wt, dy


@pytest.mark.parametrize("h,c,k", [(224, 64, 64), (112, 64, 128), (112, 128, 128)])
def test_conv_forward_statistics_and_gradients_at_benchmark_size(h, c, k):
    from renaissance_b200 import ops
    torch.backends.cudnn.allow_tf32 = False
    x, wt, dy = _tensors(h, c, k, 7 + h + k)
    g = ops.ConvGeometry(N, h, h, c, k)
    assert ops.conv_uses_tensor_cores(g, "dgrad") and ops.conv_uses_tensor_cores(g, "wgrad")
    wn = _nchw(wt)
    # forward + statistics
    y, st = ops.conv_fprop_bn_stats(g, x, wt, torch.ones(k, device="cuda"), torch.zeros(k, device="cuda"),
                                    want_sums=True)
    dx = ops.conv_dgrad(g, dy, wt)
    dw = ops.conv_wgrad(g, dy, x)
    ops.device_status()
    for i in IMAGES:
        ref_y = _nhwc(F.conv2d(_nchw(x[i:i + 1]), wn, padding=1))
        assert _rel(y[i:i + 1], ref_y) < 2e-3, f"forward, image {i}"
        ref_dx = _nhwc(F.conv_transpose2d(_nchw(dy[i:i + 1]), wn, padding=1))
        assert _rel(dx[i:i + 1], ref_dx) < 2e-3, f"data gradient, image {i}"
    # batch statistics of the half-rounded output the kernel itself wrote, in float64
    s1 = torch.zeros(k, dtype=torch.float64, device="cuda")
    s2 = torch.zeros(k, dtype=torch.float64, device="cuda")
    for i0 in range(0, N, 32):
        yd = y[i0:i0 + 32].double().reshape(-1, k)
        s1 += yd.sum(dim=0)
        s2 += (yd * yd).sum(dim=0)
    assert float((st["sum"].double() - s1).abs().max() / s1.abs().max()) < 1e-4
    assert float((st["sqsum"].double() - s2).abs().max() / s2.abs().max()) < 1e-4
    m = N * h * h
    mean = s1 / m
    inv = 1.0 / torch.sqrt(s2 / m - mean * mean + 1e-5)
    assert float((st["saved_mean"].double() - mean).abs().max()) < 1e-4 * float(mean.abs().max()) + 1e-6
    assert float((st["saved_inv_std"].double() - inv).abs().max() / inv.abs().max()) < 1e-4
    # weight gradient over the whole batch, accumulated in float64 from float32 chunks
    ref_dw = torch.zeros((k, c, 3, 3), dtype=torch.float64, device="cuda")
    for i0 in range(0, N, 16):
        ref_dw += torch.nn.grad.conv2d_weight(_nchw(x[i0:i0 + 16]), (k, c, 3, 3), _nchw(dy[i0:i0 + 16]),
                                              padding=1).double()
    assert _rel(dw, ref_dw.permute(0, 2, 3, 1)) < 2e-3


def test_first_layer_at_benchmark_size():
    """256 x 224 x 224 x 4 (3 image channels + 1 zero): forward with statistics and the weight gradient."""
    from renaissance_b200 import ops
    torch.backends.cudnn.allow_tf32 = False
    h, c, k = 224, 4, 64
    gen = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn((N, h, h, c), generator=gen, device="cuda").half()
    x[..., 3] = 0
    wt = (torch.randn((k, 3, 3, c), generator=gen, device="cuda") * (2.0 / 27) ** 0.5).half()
    dy = torch.randn((N, h, h, k), generator=gen, device="cuda").half()
    g = ops.ConvGeometry(N, h, h, c, k)
    y, st = ops.conv_fprop_bn_stats(g, x, wt, torch.ones(k, device="cuda"), torch.zeros(k, device="cuda"), want_sums=True)
    dw = ops.conv_wgrad(g, dy, x)
    ops.device_status()
    wn = _nchw(wt)
    for i in IMAGES:
        assert _rel(y[i:i + 1], _nhwc(F.conv2d(_nchw(x[i:i + 1]), wn, padding=1))) < 2e-3, f"image {i}"
    s1 = torch.zeros(k, dtype=torch.float64, device="cuda")
    for i0 in range(0, N, 32):
        s1 += y[i0:i0 + 32].double().reshape(-1, k).sum(dim=0)
    assert float((st["sum"].double() - s1).abs().max() / s1.abs().max()) < 1e-4
    ref_dw = torch.zeros((k, c, 3, 3), dtype=torch.float64, device="cuda")
    for i0 in range(0, N, 16):
        ref_dw += torch.nn.grad.conv2d_weight(_nchw(x[i0:i0 + 16]), (k, c, 3, 3), _nchw(dy[i0:i0 + 16]),
                                              padding=1).double()
    assert _rel(dw[..., :3], ref_dw.permute(0, 2, 3, 1)[..., :3]) < 2e-3


def _mask_bits_to_bool(bits, shape):
    n = 1
    for d in shape:
        n *= d
    idx = torch.arange(n, device="cuda")
    return (((bits[idx >> 3].to(torch.int32) >> (idx & 7).to(torch.int32)) & 1) == 1).reshape(shape)


@pytest.mark.parametrize("h,c", [(224, 64), (112, 128)])
def test_bn_relu_pool_forward_and_backward_at_benchmark_size(h, c):
    """bn_apply_relu_mask, the pool-fused forward, the BN+ReLU backward and the pool-fused backward on a
    256 x h x h x c activation, against torch on slabs of the batch (masks and argmax bit-exact)."""
    from renaissance_b200 import ops
    gen = torch.Generator(device="cuda").manual_seed(h + c)
    co = (torch.randn((N, h, h, c), generator=gen, device="cuda") * 1.2 + 0.1).half()
    gamma = 1 + 0.2 * torch.randn(c, generator=gen, device="cuda")
    beta = 0.1 * torch.randn(c, generator=gen, device="cuda")
    m = N * h * h
    s1 = torch.zeros(c, dtype=torch.float64, device="cuda")
    s2 = torch.zeros(c, dtype=torch.float64, device="cuda")
    for i0 in range(0, N, 32):
        d = co[i0:i0 + 32].double().reshape(-1, c)
        s1 += d.sum(dim=0)
        s2 += (d * d).sum(dim=0)
    mean64 = s1 / m
    inv64 = 1.0 / torch.sqrt(s2 / m - mean64 * mean64 + 1e-5)
    mean, inv = mean64.float(), inv64.float()
    es = gamma * inv
    eb = beta - mean * es
    relu, bits = ops.bn_apply_relu_mask(co, es, eb)
    pool, am, bits2 = ops.bn_apply_relu_mask_pool(co, es, eb)
    torch.cuda.synchronize()
    assert torch.equal(bits, bits2)
    # forward reference per slab: y = half(half(x * es) + eb), relu, mask = y > 0 (cbr_op.cpp:534-616)
    for i in IMAGES:
        yb = ((co[i].float() * es).half().float() + eb).half()
        assert torch.equal(relu[i], torch.relu(yb))
        assert torch.equal(_mask_bits_to_bool(bits[i * h * h * c // 8:(i + 1) * h * h * c // 8], (h, h, c)), yb > 0)
        ref_pool = F.max_pool2d(torch.relu(yb).float().permute(2, 0, 1)[None], 2)[0].permute(1, 2, 0).half()
        assert torch.equal(pool[i], ref_pool)
    # backward of BN + ReLU
    dy = torch.randn((N, h, h, c), generator=gen, device="cuda").half()
    dconv, dg, db = ops.bnrelu_bwd(dy, bits, co, gamma, mean, inv)
    ref_db = torch.zeros(c, dtype=torch.float64, device="cuda")
    ref_dg = torch.zeros(c, dtype=torch.float64, device="cuda")
    for i0 in range(0, N, 16):
        keep = _mask_bits_to_bool(bits[i0 * h * h * c // 8:(i0 + 16) * h * h * c // 8], (16, h, h, c))
        dym = (dy[i0:i0 + 16].float() * keep).half().double().reshape(-1, c)     # dy * mask is rounded to half
        xh = (co[i0:i0 + 16].double().reshape(-1, c) - mean64) * inv64
        ref_db += dym.sum(dim=0)
        ref_dg += (dym * xh).sum(dim=0)
    assert float((dg.double() - ref_dg).abs().max() / ref_dg.abs().max()) < 1e-4
    assert float((db.double() - ref_db).abs().max() / ref_db.abs().max()) < 1e-4
    for i in IMAGES:
        keep = _mask_bits_to_bool(bits[i * h * h * c // 8:(i + 1) * h * h * c // 8], (h, h, c))
        dym = (dy[i].float() * keep).double()
        xh = (co[i].double() - mean64) * inv64
        ref = gamma.double() * inv64 * (dym - ref_db / m - xh * ref_dg / m)
        assert _rel(dconv[i], ref) < 2e-3, f"dconv, image {i}"
    # pool-fused backward = max-pool backward, then the above
    dyp = torch.randn((N, h // 2, h // 2, c), generator=gen, device="cuda").half()
    dconv_p, dg_p, db_p = ops.bnrelu_pool_bwd(dyp, am, bits, co, gamma, mean, inv)
    dy_full = torch.empty_like(co)
    ops.maxpool2x2_bwd(dyp, am, dy_full)
    dconv_r, dg_r, db_r = ops.bnrelu_bwd(dy_full, bits, co, gamma, mean, inv)
    torch.cuda.synchronize()
    assert float((dg_p - dg_r).abs().max() / dg_r.abs().max()) < 1e-4
    assert float((db_p - db_r).abs().max() / db_r.abs().max()) < 1e-4
    for i in IMAGES:
        assert _rel(dconv_p[i], dconv_r[i].float()) < 2e-3, f"pooled dconv, image {i}"
    # the un-fused pool backward against torch on the last image (offsets beyond 2^31 bytes)
    i = N - 1
    a = relu[i].float().permute(2, 0, 1)[None].requires_grad_(True)
    F.max_pool2d(a, 2).backward(dyp[i].float().permute(2, 0, 1)[None])
    assert torch.equal(dy_full[i], a.grad[0].permute(1, 2, 0).half())


@pytest.mark.parametrize("m,c", [(75776 + 3, 64), (9472 * 4 + 1, 512), (20000, 24)])
def test_bn_apply_relu_mask_ring_and_strip_kernels_bit_exact(m, c):
    """bn_apply_relu_mask on the bulk-copy ring (tensors of four or more 1024-vector items per SM, here with rows
    past the last whole item) and on the strip kernel (channel counts the ring does not take): relu output and mask
    bits equal torch's half(half(x * s) + b) bit for bit."""
    from renaissance_b200 import ops
    gen = torch.Generator(device="cuda").manual_seed(m + c)
    x = (torch.randn((m, c), generator=gen, device="cuda") * 1.2 + 0.1).half()
    es = 0.5 + torch.rand(c, generator=gen, device="cuda")
    eb = 0.3 * torch.randn(c, generator=gen, device="cuda")
    relu, bits = ops.bn_apply_relu_mask(x, es, eb)
    yb = ((x.float() * es).half().float() + eb).half()
    assert torch.equal(relu, torch.relu(yb))
    assert torch.equal(_mask_bits_to_bool(bits, (m, c)), yb > 0)
