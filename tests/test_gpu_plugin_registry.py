"""The operator-registry adapter (renaissance_b200/plugin): the reference's
launch_cuda(node, mp, ctx, state) entries, driven the way the reference drives them --
one warm-up call outside capture, then stream capture of the node list through
g_compute_op_table on the COMP_1/2/3 streams, then CUDA-graph replay."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from conftest import rel_l2, rel_max
from gpu_util import block_inputs, dev, host

pytestmark = pytest.mark.gpu

FP32, FP16, INT8, INT32 = 0, 1, 2, 3
CBR_BWD, CBR_BWD_FIRST, SM_FWD, SM_BWD = 1, 2, 3, 4


@pytest.fixture(scope="module")
def plugin():
    from renaissance_b200 import _lib
    _lib.load()
    path = os.path.join(os.path.dirname(_lib.LIB_PATH), "libtrb200_plugin.so")
    lib = C.CDLL(path)
    lib.trbh_create.restype = C.c_void_p
    lib.trbh_last_error.restype = C.c_char_p
    lib.trbh_workspace_bytes.restype = C.c_size_t
    lib.trbh_workspace_bytes.argtypes = [C.c_void_p]
    lib.trbh_destroy.argtypes = [C.c_void_p]
    lib.trbh_add_tensor.argtypes = [C.c_void_p, C.c_int, C.c_void_p] + [C.c_int] * 5 + [C.c_longlong]
    lib.trbh_add_node.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_int), C.c_int,
                                  C.c_int, C.c_int, C.c_int, C.c_int]
    for f in (lib.trbh_warmup, lib.trbh_capture, lib.trbh_replay):
        f.argtypes = [C.c_void_p]
    return lib


def _ok(lib, rc):
    assert rc == 0, lib.trbh_last_error().decode()


def _ids(v):
    return (C.c_int * len(v))(*v), len(v)


def _add(lib, h, tid, t, shape, dtype, stride=0):
    n, hh, w, c = shape
    _ok(lib, lib.trbh_add_tensor(h, tid, t.data_ptr(), n, hh, w, c, dtype, stride))


@pytest.mark.parametrize("n,h,w,c,k,first", [(2, 14, 14, 64, 64, False), (2, 16, 16, 4, 64, True),
                                             (3, 8, 8, 16, 32, False)])
def test_cbr_bwd_node_warmup_capture_replay(orc, plugin, n, h, w, c, k, first):
    b = block_inputs(orc, 21 + c, n, h, w, c, k)
    ref = orc.cbr_bwd_amp(b["dy"], b["w"], b["gamma"], b["saved_mean"], b["saved_inv_std"], b["mask_bits"], b["x"],
                          b["conv_out"], first_layer=first)
    x0 = dev(b["x"])
    t = dict(dy=dev(b["dy"]), w=dev(b["w"]), gamma=dev(b["gamma"]), mean=dev(b["saved_mean"]),
             inv=dev(b["saved_inv_std"]), x=x0.clone(), conv_out=dev(b["conv_out"]),
             dw=torch.zeros((k, 3, 3, c), dtype=torch.float16, device="cuda"),
             dgamma=torch.zeros(k, device="cuda"), dbeta=torch.zeros(k, device="cuda"),
             bn_out=torch.zeros((n, h, w, k), dtype=torch.float16, device="cuda"))
    # the mask lives in an INT8-sized buffer of the activation's shape; only the first numel/8 bytes are used
    mask = torch.zeros(n * h * w * k, dtype=torch.uint8, device="cuda")
    mask[:b["mask_bits"].size] = dev(b["mask_bits"])
    conv_out0 = t["conv_out"].clone()
    hnd = plugin.trbh_create()
    try:
        act, out = (n, h, w, c), (n, h, w, k)
        _add(plugin, hnd, 10, t["dy"], out, FP16)
        _add(plugin, hnd, 11, t["w"], (k, 3, 3, c), FP16)
        _add(plugin, hnd, 12, t["gamma"], (1, 1, 1, k), FP32)
        _add(plugin, hnd, 13, t["mean"], (1, 1, 1, k), FP32)
        _add(plugin, hnd, 14, t["inv"], (1, 1, 1, k), FP32)
        _add(plugin, hnd, 15, mask, out, INT8)
        _add(plugin, hnd, 16, t["x"], act, FP16)
        _add(plugin, hnd, 21, t["dw"], (k, 3, 3, c), FP16)
        _add(plugin, hnd, 22, t["dgamma"], (1, 1, 1, k), FP32)
        _add(plugin, hnd, 23, t["dbeta"], (1, 1, 1, k), FP32)
        _add(plugin, hnd, 24, t["conv_out"], out, FP16)
        _add(plugin, hnd, 25, t["bn_out"], out, FP16)
        ins, n_in = _ids([10, 11, 12, 13, 14, 15, 16])
        outs, n_out = _ids([16, 21, 22, 23, 24, 25])          # out[0] = X's own id: dX in place
        _ok(plugin, plugin.trbh_add_node(hnd, CBR_BWD_FIRST if first else CBR_BWD, ins, n_in, outs, n_out, k, 3, 1, 1))
        torch.cuda.synchronize()
        _ok(plugin, plugin.trbh_warmup(hnd))
        ws_after_warmup = plugin.trbh_workspace_bytes(hnd)
        assert ws_after_warmup > 0
        t["x"].copy_(x0)
        t["conv_out"].copy_(conv_out0)
        torch.cuda.synchronize()
        _ok(plugin, plugin.trbh_capture(hnd))
        assert plugin.trbh_workspace_bytes(hnd) == ws_after_warmup      # nothing allocated while capturing
        for _ in range(2):
            t["x"].copy_(x0)
            t["conv_out"].copy_(conv_out0)
            torch.cuda.synchronize()
            _ok(plugin, plugin.trbh_replay(hnd))
            assert rel_max(host(t["dgamma"]), ref["dgamma"]) < 1e-4
            assert rel_max(host(t["dbeta"]), ref["dbeta"]) < 1e-4
            assert rel_l2(host(t["dw"]).astype(np.float32), ref["dw"].astype(np.float32)) < 2e-3
            if first:
                assert torch.equal(t["x"], x0)
            else:
                assert rel_l2(host(t["x"]).astype(np.float32), ref["dx"].astype(np.float32)) < 2e-3
    finally:
        plugin.trbh_destroy(hnd)
    from renaissance_b200 import ops
    ops.device_status()


def test_softmax_nodes_with_padded_logits_stride(orc, plugin):
    """10 classes in a feature buffer whose rows are padded to 16 (distributed_tensor.h:173-207)."""
    batch, classes, stride = 24, 10, 16
    rng = np.random.default_rng(2)
    z = (rng.standard_normal((batch, classes)) * 2).astype(np.float16)
    labels = rng.integers(0, classes, size=batch).astype(np.int32)
    ref = orc.softmax_ce_amp(z, labels, scaling=8.0, ls=0.1)
    logits = torch.zeros((batch, stride), dtype=torch.float16, device="cuda")
    logits[:, :classes] = dev(z)
    dl = torch.zeros((batch, stride), dtype=torch.float16, device="cuda")
    f = lambda v: torch.tensor([v], dtype=torch.float32, device="cuda")
    scaling, ls, loss, inv = f(8.0), f(0.1), f(0.0), f(0.0)
    bs = torch.tensor([batch], dtype=torch.int32, device="cuda")
    lab = dev(labels)
    probs = torch.zeros((batch, classes), device="cuda")
    part = torch.zeros(batch, device="cuda")
    dummy_i = torch.zeros(batch, dtype=torch.int32, device="cuda")
    dummy_f = f(0.0)
    hnd = plugin.trbh_create()
    try:
        one = (1, 1, 1, 1)
        _add(plugin, hnd, 1, logits, (batch, 1, 1, classes), FP16, stride)
        _add(plugin, hnd, 2, scaling, one, FP32)
        _add(plugin, hnd, 3, bs, one, INT32)
        _add(plugin, hnd, 4, lab, (batch, 1, 1, 1), INT32)
        _add(plugin, hnd, 5, ls, one, FP32)
        _add(plugin, hnd, 6, loss, one, FP32)
        _add(plugin, hnd, 7, inv, one, FP32)
        _add(plugin, hnd, 8, dummy_i, (batch, 1, 1, 1), INT32)
        _add(plugin, hnd, 9, probs, (batch, 1, 1, classes), FP32)
        _add(plugin, hnd, 10, dummy_f, one, FP32)
        _add(plugin, hnd, 11, part, (batch, 1, 1, 1), FP32)
        _add(plugin, hnd, 12, dl, (batch, 1, 1, classes), FP16, stride)
        ins, n_in = _ids([1, 2, 3, 4, 5])
        outs, n_out = _ids([6, 7, 8, 9, 10, 10, 11, 8, 8])
        _ok(plugin, plugin.trbh_add_node(hnd, SM_FWD, ins, n_in, outs, n_out, 0, 0, 0, 0))
        ins, n_in = _ids([12, 9, 7, 2, 4, 5])
        outs, n_out = _ids([12])
        _ok(plugin, plugin.trbh_add_node(hnd, SM_BWD, ins, n_in, outs, n_out, 0, 0, 0, 0))
        _ok(plugin, plugin.trbh_warmup(hnd))
        _ok(plugin, plugin.trbh_capture(hnd))
        _ok(plugin, plugin.trbh_replay(hnd))
        assert abs(float(loss) - ref["loss"]) < 2e-5 and float(inv) == pytest.approx(1 / batch)
        assert np.abs(host(probs) - ref["probs"]).max() < 5e-6
        assert rel_l2(host(dl[:, :classes]).astype(np.float32), ref["dlogits"].astype(np.float32)) < 2e-3
        assert float(dl[:, classes:].abs().max()) == 0.0
    finally:
        plugin.trbh_destroy(hnd)


def test_unsupported_shape_surfaces_as_an_exception_text(plugin):
    """A non-zero C-ABI status becomes the reference's exception (here: its message)."""
    hnd = plugin.trbh_create()
    try:
        buf = torch.zeros(4096, dtype=torch.float16, device="cuda")
        for tid in (10, 11, 12, 13, 14, 15, 16, 21, 22, 23, 24, 25):
            _add(plugin, hnd, tid, buf, (1, 4, 4, 12), FP16)          # k = 12 is not a multiple of 8
        ins, n_in = _ids([10, 11, 12, 13, 14, 15, 16])
        outs, n_out = _ids([16, 21, 22, 23, 24, 25])
        _ok(plugin, plugin.trbh_add_node(hnd, CBR_BWD, ins, n_in, outs, n_out, 12, 3, 1, 1))
        assert plugin.trbh_warmup(hnd) == -1
        msg = plugin.trbh_last_error().decode()
        assert "CBR_AMP_BWD" in msg and "trb200 status" in msg
    finally:
        plugin.trbh_destroy(hnd)
