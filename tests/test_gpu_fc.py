"""Classifier kernels: FC forward / backward on the library's own tensor-core GEMMs with bias, ReLU and dropout
(FC_AMP_FWD / FC_AMP_BWD, fc_op.cpp:259-480) against the oracle's restatement of the reference's CPU operator
(fc_op.cpp:802-898) and, at the VGG16 sizes, against torch in float32."""
import numpy as np
import pytest
import torch

from conftest import rel_l2, rel_max
from gpu_util import dev, host

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("batch,in_f,out_f", [(4, 64, 64), (7, 128, 256), (32, 512, 128), (256, 2048, 256),
                                               (5, 256, 1024), (130, 320 * 4, 512), (3, 8, 8), (300, 200, 1000),
                                               (257, 72, 264), (64, 6000, 40)])
def test_fc_matches_oracle(orc, batch, in_f, out_f):
    from renaissance_b200 import ops
    rng = np.random.default_rng(batch + in_f)
    x = rng.standard_normal((batch, in_f)).astype(np.float16)
    w = (rng.standard_normal((out_f, in_f)) * np.sqrt(2.0 / in_f)).astype(np.float16)
    b = (0.1 * rng.standard_normal(out_f)).astype(np.float32)
    dy = rng.standard_normal((batch, out_f)).astype(np.float16)
    y_ref = orc.fc_fwd(x.astype(np.float32), w.astype(np.float32), b)
    dx_ref, dw_ref, db_ref = orc.fc_bwd(dy.astype(np.float32), w.astype(np.float32), x.astype(np.float32))
    y = ops.fc_amp_fwd(dev(x), dev(w), dev(b))
    dx, dw, db = ops.fc_amp_bwd(dev(dy), dev(w), dev(x))
    ops.device_status()
    assert rel_l2(host(y).astype(np.float32), y_ref) < 2e-3
    assert rel_l2(host(dx).astype(np.float32), dx_ref) < 2e-3
    assert rel_l2(host(dw).astype(np.float32), dw_ref) < 2e-3
    assert rel_max(host(db), db_ref) < 1e-4                       # a per-channel reduction: 1e-4 relative
    # ReLU folded in: bit-identical to the plain output passed through max(., 0)
    yr = ops.fc_amp_fwd(dev(x), dev(w), dev(b), relu=True)
    assert torch.equal(yr, torch.relu(y))
    # float dW, as the reference's operator writes it
    dwf = torch.empty((out_f, in_f), dtype=torch.float32, device="cuda")
    ops.fc_amp_bwd(dev(dy), dev(w), dev(x), dw=dwf, want_dx=False)
    assert rel_l2(host(dwf), dw_ref) < 1e-4 and torch.equal(dwf.half(), dw)
    # twice the same: reproducible
    dx2, dw2, db2 = ops.fc_amp_bwd(dev(dy), dev(w), dev(x))
    assert torch.equal(dx, dx2) and torch.equal(dw, dw2) and torch.equal(db, db2)


def test_dropout_is_a_counter_based_mask_and_its_backward_needs_only_the_output():
    from renaissance_b200 import ops
    batch, in_f, out_f, p = 256, 512, 4096, 0.5
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn((batch, in_f), generator=g, device="cuda").half()
    w = (torch.randn((out_f, in_f), generator=g, device="cuda") * (2.0 / in_f) ** 0.5).half()
    b = torch.zeros(out_f, device="cuda")
    plain = ops.fc_amp_fwd(x, w, b, relu=True)
    d1 = ops.fc_amp_fwd(x, w, b, relu=True, dropout_p=p, seed=123, offset=7)
    d2 = ops.fc_amp_fwd(x, w, b, relu=True, dropout_p=p, seed=123, offset=7)
    d3 = ops.fc_amp_fwd(x, w, b, relu=True, dropout_p=p, seed=123, offset=8)
    assert torch.equal(d1, d2) and not torch.equal(d1, d3)                     # same counter, same mask
    kept = d1 != 0
    live = plain > 0
    assert bool((kept <= live).all())                                          # only live elements survive
    rate = float(kept[live].float().mean())
    assert abs(rate - (1 - p)) < 5e-3                                          # about half of ~500 k live elements kept
    assert torch.equal(d1[kept], (plain[kept].float() * 2.0).half())           # kept ones scaled by 1 / (1 - p)
    # the two masks of different counters are independent: they agree on about half of the live elements
    kept3 = d3 != 0
    agree = float((kept[live] == kept3[live]).float().mean())
    assert abs(agree - 0.5) < 5e-3
    # columns and rows are not correlated with the mask
    assert float(kept.float().mean(dim=0).std()) < 0.05 and float(kept.float().mean(dim=1).std()) < 0.05
    # backward from the output alone
    da = torch.randn((batch, out_f), generator=g, device="cuda").half()
    dz = ops.fc_act_bwd(da, d1, scale=1.0 / (1 - p))
    expect = torch.where(kept, (da.float() * 2.0).half(), torch.zeros_like(da))
    assert torch.equal(dz, expect)
    inplace = da.clone()
    ops.fc_act_bwd(inplace, d1, dz=inplace, scale=1.0 / (1 - p))
    assert torch.equal(inplace, expect)
    # the same folded into the next layer's backward: dx of a layer whose input is d1
    w2 = (torch.randn((1024, out_f), generator=g, device="cuda") * (2.0 / out_f) ** 0.5).half()
    dy2 = torch.randn((batch, 1024), generator=g, device="cuda").half()
    dx_plain, _, _ = ops.fc_amp_bwd(dy2, w2, d1)
    dx_fused, _, _ = ops.fc_amp_bwd(dy2, w2, d1, act=d1, act_scale=1.0 / (1 - p))
    assert torch.equal(dx_fused, ops.fc_act_bwd(dx_plain, d1, scale=1.0 / (1 - p)))


@pytest.mark.parametrize("in_f,out_f", [(25088, 4096), (4096, 4096), (4096, 1024)])
def test_vgg16_classifier_sizes_against_torch_float32(in_f, out_f):
    from renaissance_b200 import ops
    batch = 256
    g = torch.Generator(device="cuda").manual_seed(in_f)
    x = torch.randn((batch, in_f), generator=g, device="cuda").half()
    w = (torch.randn((out_f, in_f), generator=g, device="cuda") * (2.0 / in_f) ** 0.5).half()
    b = 0.1 * torch.randn(out_f, generator=g, device="cuda")
    dy = torch.randn((batch, out_f), generator=g, device="cuda").half()
    y = ops.fc_amp_fwd(x, w, b)
    dx, dw, db = ops.fc_amp_bwd(dy, w, x)
    ops.device_status()
    torch.backends.cuda.matmul.allow_tf32 = False
    rel = lambda a, r: float((a.double() - r.double()).norm() / r.double().norm())
    assert rel(y, x.float() @ w.float().t() + b) < 2e-3
    assert rel(dx, dy.float() @ w.float()) < 2e-3
    assert rel(dw, dy.float().t() @ x.float()) < 2e-3
    ref_db = dy.double().sum(dim=0)
    assert float((db.double() - ref_db).abs().max() / ref_db.abs().max()) < 1e-4


def test_unsupported_width_is_refused():
    from renaissance_b200 import _lib
    lib = _lib.load()
    assert lib.trb200_fc_amp_workspace_bytes(8, 4096, 1001) == 0          # rows must be whole 16-byte vectors
    x = torch.zeros((8, 4096), dtype=torch.float16, device="cuda")
    w = torch.zeros((1001, 4096), dtype=torch.float16, device="cuda")
    y = torch.zeros((8, 1001), dtype=torch.float16, device="cuda")
    ws = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    rc = lib.trb200_fc_amp_fwd(x.data_ptr(), w.data_ptr(), None, y.data_ptr(), 8, 4096, 1001, 0, 0.0, 0, 0,
                               ws.data_ptr(), ws.numel(), None)
    assert rc == _lib.ERR_UNSUPPORTED
    # a workspace that is too small is refused too
    rc = lib.trb200_fc_amp_fwd(x.data_ptr(), w.data_ptr(), None, y.data_ptr(), 8, 4096, 1000, 0, 0.0, 0, 0,
                               ws.data_ptr(), 16, None)
    assert rc == _lib.ERR_WORKSPACE


@pytest.mark.parametrize("batch,in_f,out_f", [(256, 2048, 1000), (7, 128, 256), (130, 1280, 512)])
def test_fc_bfloat16_against_torch_float32(batch, in_f, out_f):
    """The classifier of a bfloat16 network (ResNet-50's 2048 -> 1000 head): forward with bias, data gradient, weight
    gradient in bfloat16 and in float, bias gradient; against float32 torch on the bfloat16-rounded operands.
    bfloat16 keeps 8 significant bits: 4e-3 relative L2 on its outputs."""
    from renaissance_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(batch + out_f)
    x = torch.randn((batch, in_f), generator=g, device="cuda").bfloat16()
    w = (torch.randn((out_f, in_f), generator=g, device="cuda") * (2.0 / in_f) ** 0.5).bfloat16()
    b = 0.1 * torch.randn(out_f, generator=g, device="cuda")
    dy = torch.randn((batch, out_f), generator=g, device="cuda").bfloat16()
    y = ops.fc_amp_fwd(x, w, b)
    dx, dw, db = ops.fc_amp_bwd(dy, w, x)
    dwf = torch.empty((out_f, in_f), dtype=torch.float32, device="cuda")
    ops.fc_amp_bwd(dy, w, x, dw=dwf, want_dx=False)
    ops.device_status()
    assert y.dtype == torch.bfloat16 and dx.dtype == torch.bfloat16 and dw.dtype == torch.bfloat16

    def rel(a, ref):
        return float((a.float() - ref).norm() / ref.norm())

    y_ref = x.float() @ w.float().t() + b
    assert rel(y, y_ref) < 4e-3
    assert rel(dx, dy.float() @ w.float()) < 4e-3
    dw_ref = dy.float().t() @ x.float()
    assert rel(dw, dw_ref) < 4e-3 and rel(dwf, dw_ref) < 1e-4
    db_ref = dy.float().sum(dim=0)
    assert float((db - db_ref).abs().max() / db_ref.abs().max()) < 1e-4
    assert torch.equal(ops.fc_amp_fwd(x, w, b, relu=True), torch.relu(y))
