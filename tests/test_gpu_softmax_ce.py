"""Softmax-CE forward / backward / fused kernels against the CPU oracle and goldens."""
import numpy as np
import pytest
import torch

from conftest import golden, rel_l2
from gpu_util import dev, host

pytestmark = pytest.mark.gpu


def _scalars(scaling, ls):
    return (torch.tensor([scaling], dtype=torch.float32, device="cuda"),
            torch.tensor([ls], dtype=torch.float32, device="cuda"))


def _check(out, ref, want_probs, batch):
    if want_probs:
        assert np.abs(host(out["probs"]) - ref["probs"]).max() < 5e-6
        # bit-exact argmax
        assert np.array_equal(host(out["probs"]).argmax(axis=1), ref["probs"].argmax(axis=1))
    assert np.abs(host(out["loss_partial"]) - ref["loss_partial"]).max() < 2e-5 / batch + 1e-7
    assert abs(float(out["loss"]) - ref["loss"]) < 2e-5
    assert float(out["inv_scaling"]) == pytest.approx(1.0 / batch)


@pytest.mark.parametrize("batch,classes,ls,scaling", [
    (1, 1, 0.0, 1.0), (3, 2, 0.0, 1.0), (8, 10, 0.0, 1.0), (5, 16, 0.1, 8.0), (64, 1000, 0.0, 1024.0),
    (64, 1000, 0.1, 1024.0), (33, 257, 0.1, 2.0), (16, 2048, 0.05, 1.0), (9, 2056, 0.1, 1.0),
    (6, 10000, 0.0, 1024.0), (4, 32000, 0.1, 1024.0), (3, 4999, 0.1, 1.0),
    # every (threads, vectors per thread) variant of the register-resident row kernel, plus a ragged persistent loop
    (5, 2560, 0.1, 4.0), (4, 6000, 0.0, 1024.0), (4, 8000, 0.1, 1.0), (3, 12000, 0.0, 16.0), (3, 16000, 0.1, 1.0),
    (3, 24000, 0.0, 1024.0), (2, 32768, 0.1, 1.0), (700, 4096, 0.0, 1024.0), (3000, 1000, 0.1, 1024.0),
    # more rows than persistent blocks: the ring of row buffers wraps several times
    (2000, 10000, 0.0, 1024.0), (700, 16000, 0.1, 1024.0), (400, 32000, 0.0, 1024.0)])
def test_fused_and_split_nodes_match_oracle(orc, batch, classes, ls, scaling):
    from renaissance_b200 import ops
    rng = np.random.default_rng(batch * 131 + classes)
    z = (rng.standard_normal((batch, classes)) * 2.0).astype(np.float16)
    labels = rng.integers(0, classes, size=batch).astype(np.int32)
    ref = orc.softmax_ce_amp(z, labels, scaling=scaling, ls=ls)
    sc, lsd = _scalars(scaling, ls)
    zd, ld = dev(z), dev(labels)
    # fused: one pass
    fused = ops.softmax_ce_amp_fused(zd, ld, sc, lsd, want_probs=True)
    torch.cuda.synchronize()
    _check(fused, ref, True, batch)
    assert rel_l2(host(fused["dlogits"]).astype(np.float32), ref["dlogits"].astype(np.float32)) < 2e-3
    # fused without probs (long rows then keep exp(z - max) as half between the sweeps): same gradient to half precision
    lean = ops.softmax_ce_amp_fused(zd, ld, sc, lsd, want_probs=False)
    assert lean["probs"] is None
    assert rel_l2(host(lean["dlogits"]).astype(np.float32), ref["dlogits"].astype(np.float32)) < 2e-3
    assert abs(float(lean["loss"]) - ref["loss"]) < 2e-5
    # the reference's two nodes
    fwd = ops.softmax_ce_amp_fwd(zd, ld, lsd)
    _check(fwd, ref, True, batch)
    d = ops.softmax_ce_amp_bwd(fwd["probs"], ld, sc, fwd["inv_scaling"], lsd)
    assert rel_l2(host(d).astype(np.float32), ref["dlogits"].astype(np.float32)) < 2e-3
    # labels are read, never written
    assert np.array_equal(host(ld), labels)


def test_padded_row_stride(orc):
    """Logits live in a feature buffer whose row stride is padded to a multiple of 8
    (10 classes -> stride 16)."""
    from renaissance_b200 import _lib, ops
    import ctypes as C
    batch, classes, stride = 12, 10, 16
    rng = np.random.default_rng(5)
    z = (rng.standard_normal((batch, classes)) * 2).astype(np.float16)
    labels = rng.integers(0, classes, size=batch).astype(np.int32)
    ref = orc.softmax_ce_amp(z, labels, scaling=4.0, ls=0.1)
    zp = torch.full((batch, stride), 7.0, dtype=torch.float16, device="cuda")
    zp[:, :classes] = dev(z)
    dl = torch.full((batch, stride), -3.0, dtype=torch.float16, device="cuda")
    sc, lsd = _scalars(4.0, 0.1)
    part = torch.empty(batch, device="cuda")
    loss = torch.empty(1, device="cuda")
    inv = torch.empty(1, device="cuda")
    lib = _lib.load()
    ld = dev(labels)
    _lib.check(lib.trb200_softmax_ce_fused(zp.data_ptr(), stride, ld.data_ptr(), sc.data_ptr(), lsd.data_ptr(),
                                           None, 0, dl.data_ptr(), stride, part.data_ptr(), loss.data_ptr(),
                                           inv.data_ptr(), batch, classes, None))
    torch.cuda.synchronize()
    assert rel_l2(host(dl[:, :classes]).astype(np.float32), ref["dlogits"].astype(np.float32)) < 2e-3
    assert float((dl[:, classes:] + 3.0).abs().max()) == 0.0     # padding untouched
    assert abs(float(loss) - ref["loss"]) < 2e-5


@pytest.mark.parametrize("name", ["softmax_fp16_1000", "softmax_fp16_ls"])
def test_matches_golden(name):
    from renaissance_b200 import ops
    g = golden(name)
    batch = int(g["params"][0])
    sc, lsd = _scalars(float(g["scaling"]), float(g["ls"]))
    out = ops.softmax_ce_amp_fused(dev(g["logits"].astype(np.float16)), dev(g["labels"]), sc, lsd, want_probs=True)
    assert abs(float(out["loss"]) - float(g["loss"])) < 5e-5
    assert np.abs(host(out["probs"]) - g["probs"]).max() < 5e-6
    assert np.array_equal(host(out["probs"]).argmax(axis=1).astype(np.int32), g["pred"])
    assert rel_l2(host(out["dlogits"]).astype(np.float32), g["dlogits"]) < 1e-3


def test_large_sweep_point_properties():
    """N=4096 x C=32000 (a point of the kernel sweep): rows of the gradient sum to
    zero up to half rounding, the label entry is the only negative one for ls=0, and
    the loss equals mean(-log(softmax_y + 1e-8)) taken with torch in float32 (the
    1e-8 inside the log is the reference's and is visible at p_y ~ 1e-6)."""
    from renaissance_b200 import ops
    batch, classes = 4096, 32000
    g = torch.Generator(device="cuda").manual_seed(1)
    z = (torch.randn((batch, classes), generator=g, device="cuda") * 2).half()
    labels = torch.randint(0, classes, (batch,), generator=g, device="cuda", dtype=torch.int32)
    sc, lsd = _scalars(1024.0, 0.0)
    out = ops.softmax_ce_amp_fused(z, labels, sc, lsd)
    rows = torch.arange(batch, device="cuda")
    p_y = torch.softmax(z.float(), dim=1)[rows, labels.long()]
    ref_loss = (-torch.log(p_y + 1e-8)).double().mean()
    assert abs(float(out["loss"]) - float(ref_loss)) < 1e-4
    d = out["dlogits"].float()
    assert bool((d[rows, labels.long()] < 0).all())
    d[rows, labels.long()] = 0
    assert bool((d >= 0).all())
    full = out["dlogits"].double().sum(dim=1)
    assert float(full.abs().max()) < 1024.0 / batch * 2e-2


@pytest.mark.parametrize("classes,stride", [(10, 16), (1000, 1008), (2056, 2064), (10000, 10008), (4999, 5000)])
@pytest.mark.parametrize("want_probs", [False, True])
def test_labels_out_of_range_touch_nothing(classes, stride, want_probs):
    """Labels -1 and `classes` (an ignore index, a corrupt batch) match no class: no access goes through them.  The
    d_logits buffer has a wider row stride with sentinel padding; the padding and the rows of the valid labels must
    come out exactly as in a run in which the bad rows hold a valid label, and the bad rows must be the plain
    (p - ls/C) * scale gradient.  Every row kernel is reached by one of the shapes."""
    from renaissance_b200 import _lib
    batch = 16
    rng = np.random.default_rng(classes)
    z = (rng.standard_normal((batch, classes)) * 2).astype(np.float16)
    labels = rng.integers(0, classes, size=batch).astype(np.int32)
    bad = labels.copy()
    bad[3], bad[7], bad[12] = -1, classes, 2**31 - 1
    zp = torch.full((batch, stride), 0.5, dtype=torch.float16, device="cuda")
    zp[:, :classes] = dev(z)
    sc, lsd = _scalars(8.0, 0.1)
    lib = _lib.load()

    def run(lab):
        dl = torch.full((batch + 2, stride), -3.0, dtype=torch.float16, device="cuda")   # a guard row either side
        probs = torch.full((batch, classes), -1.0, device="cuda") if want_probs else None
        part = torch.empty(batch, device="cuda")
        loss = torch.empty(1, device="cuda")
        inv = torch.empty(1, device="cuda")
        ld = dev(lab)
        _lib.check(lib.trb200_softmax_ce_fused(zp.data_ptr(), stride, ld.data_ptr(), sc.data_ptr(), lsd.data_ptr(),
                                               probs.data_ptr() if want_probs else None, classes if want_probs else 0,
                                               dl[1:].data_ptr(), stride, part.data_ptr(), loss.data_ptr(),
                                               inv.data_ptr(), batch, classes, None))
        torch.cuda.synchronize()
        return dl, part, loss

    dl_ok, part_ok, _ = run(labels)
    dl_bad, part_bad, loss_bad = run(bad)
    assert float((dl_bad[0] + 3.0).abs().max()) == 0.0 and float((dl_bad[-1] + 3.0).abs().max()) == 0.0
    assert float((dl_bad[1:-1, classes:] + 3.0).abs().max()) == 0.0                       # padding untouched
    good = np.array([i for i in range(batch) if i not in (3, 7, 12)])
    assert torch.equal(dl_bad[1:-1][good], dl_ok[1:-1][good])                             # neighbours unchanged
    assert torch.equal(part_bad[good], part_ok[good])
    p = torch.softmax(zp[:, :classes].float(), dim=1)
    for r in (3, 7, 12):
        expect = (p[r] - 0.1 / classes) * (8.0 / batch)
        got = dl_bad[1 + r, :classes].float()
        assert float((got - expect).abs().max()) < 2e-3 * float(expect.abs().max()) + 1e-6
        assert bool(torch.isfinite(part_bad[r]))
    assert bool(torch.isfinite(loss_bad).all())
    # the two separate nodes: same rule
    ld = dev(bad)
    pr = torch.empty((batch, classes), device="cuda")
    part = torch.empty(batch, device="cuda")
    loss = torch.empty(1, device="cuda")
    inv = torch.empty(1, device="cuda")
    _lib.check(lib.trb200_softmax_ce_fwd(zp.data_ptr(), stride, ld.data_ptr(), lsd.data_ptr(), pr.data_ptr(), classes,
                                         part.data_ptr(), loss.data_ptr(), inv.data_ptr(), batch, classes, None))
    d2 = torch.full((batch, stride), -3.0, dtype=torch.float16, device="cuda")
    _lib.check(lib.trb200_softmax_ce_bwd(pr.data_ptr(), classes, ld.data_ptr(), sc.data_ptr(), inv.data_ptr(),
                                         lsd.data_ptr(), d2.data_ptr(), stride, batch, classes, None))
    torch.cuda.synchronize()
    assert float((d2[:, classes:] + 3.0).abs().max()) == 0.0
    assert bool(torch.isfinite(part).all())
    assert float((d2[:, :classes].float() - dl_bad[1:-1, :classes].float()).abs().max()) < 2e-3


def test_loss_counters_belong_to_streams():
    """The fused kernels finish the loss with a counter kept per (device, stream).  More streams than counters, all in
    flight at once, still give every call its own loss."""
    from renaissance_b200 import ops
    batch, classes = 512, 1000
    g = torch.Generator(device="cuda").manual_seed(3)
    sc, lsd = _scalars(1024.0, 0.0)
    streams = [torch.cuda.Stream() for _ in range(70)]
    zs = [(torch.randn((batch, classes), generator=g, device="cuda") * (1.0 + 0.02 * i)).half() for i in range(70)]
    labels = torch.randint(0, classes, (batch,), generator=g, device="cuda", dtype=torch.int32)
    torch.cuda.synchronize()
    outs = []
    for rep in range(2):
        outs = [ops.softmax_ce_amp_fused(z, labels, sc, lsd, stream=st) for z, st in zip(zs, streams)]
    torch.cuda.synchronize()
    rows = torch.arange(batch, device="cuda")
    for z, o in zip(zs, outs):
        p_y = torch.softmax(z.float(), dim=1)[rows, labels.long()]
        ref = float((-torch.log(p_y + 1e-8)).double().mean())
        assert abs(float(o["loss"]) - ref) < 1e-4
