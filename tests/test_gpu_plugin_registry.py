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


CBR_FWD, FC_FWD, FC_BWD = 5, 6, 7
R_BN_STATS_AR, R_SUM_AR, R_MEAN_AR, R_CHECK_NAN, R_GRAD_SCALING = 1, 2, 3, 4, 5


def _range_api(lib):
    lib.trbh_add_range_node.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_ulonglong, C.c_ulonglong, C.POINTER(C.c_int),
                                        C.c_int]
    lib.trbh_set_rank.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    lib.trbh_nccl_unique_id.argtypes = [C.c_void_p]
    lib.trbh_nccl_init.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    lib.trbh_nccl_destroy.argtypes = [C.c_void_p]
    return lib


def test_cbr_fwd_node_keeps_the_reference_layout(orc, plugin):
    """CBR_AMP_FWD through the registry: eq_scale / eq_bias land in the first 2*K floats of the bn_output buffer
    (cbr_op.cpp:1105-1108), the running statistics go prev -> next, and the outputs are what the backward node
    reads (conv_output, saved statistics, bit-packed mask)."""
    n, h, w, c, k = 2, 12, 12, 64, 64
    rng = np.random.default_rng(9)
    x = rng.standard_normal((n, h, w, c)).astype(np.float16)
    wt = (rng.standard_normal((k, 3, 3, c)) * np.sqrt(2.0 / (9 * c))).astype(np.float16)
    gamma = (1 + 0.2 * rng.standard_normal(k)).astype(np.float32)
    beta = (0.2 * rng.standard_normal(k)).astype(np.float32)
    rm0 = (0.1 * rng.standard_normal(k)).astype(np.float32)
    rv0 = (1 + 0.1 * rng.random(k)).astype(np.float32)
    rm, rv = rm0.copy(), rv0.copy()
    ref = orc.cbr_fwd_amp(x, wt, gamma, beta, running_mean=rm, running_var=rv, stats_from_half=True)
    t = dict(x=dev(x), w=dev(wt), gamma=dev(gamma), beta=dev(beta), pm=dev(rm0), pv=dev(rv0),
             conv=torch.zeros((n, h, w, k), dtype=torch.float16, device="cuda"), s1=torch.zeros(k, device="cuda"),
             s2=torch.zeros(k, device="cuda"), bn_out=torch.zeros((n, h, w, k), dtype=torch.float16, device="cuda"),
             mean=torch.zeros(k, device="cuda"), inv=torch.zeros(k, device="cuda"),
             relu=torch.zeros((n, h, w, k), dtype=torch.float16, device="cuda"),
             mask=torch.zeros(n * h * w * k, dtype=torch.uint8, device="cuda"), nm=torch.zeros(k, device="cuda"),
             nv=torch.zeros(k, device="cuda"))
    hnd = plugin.trbh_create()
    try:
        act, out, vec = (n, h, w, c), (n, h, w, k), (1, 1, 1, k)
        for tid, key, shape, dt in ((1, "x", act, FP16), (2, "w", (k, 3, 3, c), FP16), (3, "gamma", vec, FP32),
                                    (4, "beta", vec, FP32), (5, "pm", vec, FP32), (6, "pv", vec, FP32),
                                    (10, "conv", out, FP16), (11, "s1", vec, FP32), (12, "s2", vec, FP32),
                                    (13, "bn_out", out, FP16), (14, "mean", vec, FP32), (15, "inv", vec, FP32),
                                    (16, "relu", out, FP16), (17, "mask", out, INT8), (18, "nm", vec, FP32),
                                    (19, "nv", vec, FP32)):
            _add(plugin, hnd, tid, t[key], shape, dt)
        ins, n_in = _ids([1, 2, 3, 4, 5, 6])
        outs, n_out = _ids([10, 11, 12, 13, 14, 15, 16, 17, 18, 19])
        _ok(plugin, plugin.trbh_add_node(hnd, CBR_FWD, ins, n_in, outs, n_out, k, 3, 1, 1))
        _ok(plugin, plugin.trbh_warmup(hnd))
        _ok(plugin, plugin.trbh_capture(hnd))
        _ok(plugin, plugin.trbh_replay(hnd))
        assert rel_l2(host(t["conv"]).astype(np.float32), ref["conv_out"].astype(np.float32)) < 2e-3
        assert np.abs(host(t["mean"]) - ref["saved_mean"]).max() < 1e-3
        assert rel_max(host(t["inv"]), ref["saved_inv_std"]) < 1e-3
        eq = t["bn_out"].view(torch.float32).reshape(-1)[:2 * k]            # eq_scale then eq_bias
        assert rel_max(host(eq[:k]), gamma * ref["saved_inv_std"]) < 1e-3
        assert np.abs(host(eq[k:]) - (beta - ref["saved_mean"] * gamma * ref["saved_inv_std"])).max() < 2e-3
        assert np.abs(host(t["nm"]) - rm).max() < 1e-3 and rel_max(host(t["nv"]), rv) < 1e-3      # next = f(prev)
        assert torch.equal(t["pm"], dev(rm0)) and torch.equal(t["pv"], dev(rv0))                  # prev untouched
        # ReLU output and mask are exactly the apply stage of the kernel's own conv output and constants
        yb = ((t["conv"].float() * eq[:k]).half().float() + eq[k:]).half()
        assert torch.equal(t["relu"], torch.relu(yb))
        bits = host(t["mask"])[: n * h * w * k // 8]
        assert np.array_equal(orc.mask_unpack(bits, n * h * w * k).reshape(n, h, w, k), host(yb > 0).astype(np.uint8))
    finally:
        plugin.trbh_destroy(hnd)


def test_fused_softmax_pair_on_a_patched_graph(orc, plugin):
    """The forward node of a patched graph lists d_logits as output [9] and the backward node lists the logits as
    input [6]: the forward launcher then does both in one pass and the backward launcher launches nothing."""
    from renaissance_b200 import ops
    batch, classes = 64, 1000
    rng = np.random.default_rng(4)
    z = (rng.standard_normal((batch, classes)) * 2).astype(np.float16)
    labels = rng.integers(0, classes, size=batch).astype(np.int32)
    ref = orc.softmax_ce_amp(z, labels, scaling=1024.0, ls=0.0)
    logits, lab = dev(z), dev(labels)
    dl = torch.zeros((batch, classes), dtype=torch.float16, device="cuda")
    f = lambda v: torch.tensor([v], dtype=torch.float32, device="cuda")
    scaling, ls, loss, inv = f(1024.0), f(0.0), f(0.0), f(0.0)
    bs = torch.tensor([batch], dtype=torch.int32, device="cuda")
    probs = torch.zeros((batch, classes), device="cuda")
    part = torch.zeros(batch, device="cuda")
    dummy_i = torch.zeros(batch, dtype=torch.int32, device="cuda")
    dummy_f = f(0.0)
    hnd = plugin.trbh_create()
    try:
        one = (1, 1, 1, 1)
        for tid, tt, shape, dt in ((1, logits, (batch, 1, 1, classes), FP16), (2, scaling, one, FP32), (3, bs, one, INT32),
                                   (4, lab, (batch, 1, 1, 1), INT32), (5, ls, one, FP32), (6, loss, one, FP32),
                                   (7, inv, one, FP32), (8, dummy_i, (batch, 1, 1, 1), INT32),
                                   (9, probs, (batch, 1, 1, classes), FP32), (10, dummy_f, one, FP32),
                                   (11, part, (batch, 1, 1, 1), FP32), (12, dl, (batch, 1, 1, classes), FP16)):
            _add(plugin, hnd, tid, tt, shape, dt)
        ins, n_in = _ids([1, 2, 3, 4, 5])
        outs, n_out = _ids([6, 7, 8, 9, 10, 10, 11, 8, 8, 12])           # [9] = d_logits: the patched forward node
        _ok(plugin, plugin.trbh_add_node(hnd, SM_FWD, ins, n_in, outs, n_out, 0, 0, 0, 0))
        ins, n_in = _ids([12, 9, 7, 2, 4, 5, 1])                         # [6] = logits: the patched backward node
        outs, n_out = _ids([12])
        _ok(plugin, plugin.trbh_add_node(hnd, SM_BWD, ins, n_in, outs, n_out, 0, 0, 0, 0))
        before = ops.kernel_launch_count()
        _ok(plugin, plugin.trbh_warmup(hnd))
        assert ops.kernel_launch_count() - before == 1                    # one kernel for both nodes
        _ok(plugin, plugin.trbh_capture(hnd))
        dl.zero_()
        torch.cuda.synchronize()
        _ok(plugin, plugin.trbh_replay(hnd))
        assert abs(float(loss) - ref["loss"]) < 2e-5 and float(inv) == pytest.approx(1 / batch)
        assert rel_l2(host(dl).astype(np.float32), ref["dlogits"].astype(np.float32)) < 2e-3
        assert float(probs.abs().max()) == 0.0          # the probabilities are not materialised in the fused form
    finally:
        plugin.trbh_destroy(hnd)


def test_fc_nodes_write_float_weight_gradients(orc, plugin):
    batch, in_f, out_f = 32, 256, 128
    rng = np.random.default_rng(8)
    x = rng.standard_normal((batch, in_f)).astype(np.float16)
    w = (rng.standard_normal((out_f, in_f)) * np.sqrt(2.0 / in_f)).astype(np.float16)
    b = (0.1 * rng.standard_normal(out_f)).astype(np.float32)
    dy = rng.standard_normal((batch, out_f)).astype(np.float16)
    y_ref = orc.fc_fwd(x.astype(np.float32), w.astype(np.float32), b)
    dx_ref, dw_ref, db_ref = orc.fc_bwd(dy.astype(np.float32), w.astype(np.float32), x.astype(np.float32))
    t = dict(x=dev(x), w=dev(w), b=dev(b), dy=dev(dy), y=torch.zeros((batch, out_f), dtype=torch.float16, device="cuda"),
             dx=torch.zeros((batch, in_f), dtype=torch.float16, device="cuda"),
             dw=torch.zeros((out_f, in_f), device="cuda"), db=torch.zeros(out_f, device="cuda"))
    hnd = plugin.trbh_create()
    try:
        _add(plugin, hnd, 1, t["x"], (batch, 1, 1, in_f), FP16)
        _add(plugin, hnd, 2, t["w"], (out_f, 1, 1, in_f), FP16)
        _add(plugin, hnd, 3, t["b"], (1, 1, 1, out_f), FP32)
        _add(plugin, hnd, 4, t["y"], (batch, 1, 1, out_f), FP16)
        _add(plugin, hnd, 5, t["dy"], (batch, 1, 1, out_f), FP16)
        _add(plugin, hnd, 6, t["dx"], (batch, 1, 1, in_f), FP16)
        _add(plugin, hnd, 7, t["dw"], (out_f, 1, 1, in_f), FP32)
        _add(plugin, hnd, 8, t["db"], (1, 1, 1, out_f), FP32)
        ins, n_in = _ids([1, 2, 3])
        outs, n_out = _ids([4])
        _ok(plugin, plugin.trbh_add_node(hnd, FC_FWD, ins, n_in, outs, n_out, out_f, 1, 0, 0))
        ins, n_in = _ids([5, 2, 3, 1])                                    # [dy, w, bias, x]: x is the last input
        outs, n_out = _ids([6, 7, 8])
        _ok(plugin, plugin.trbh_add_node(hnd, FC_BWD, ins, n_in, outs, n_out, out_f, 1, 0, 0))
        _ok(plugin, plugin.trbh_warmup(hnd))
        _ok(plugin, plugin.trbh_capture(hnd))
        for key in ("y", "dx", "dw", "db"):
            t[key].zero_()
        torch.cuda.synchronize()
        _ok(plugin, plugin.trbh_replay(hnd))
        assert rel_l2(host(t["y"]).astype(np.float32), y_ref) < 2e-3
        assert rel_l2(host(t["dx"]).astype(np.float32), dx_ref) < 2e-3
        assert rel_l2(host(t["dw"]), dw_ref) < 1e-4                       # float dW, as FC_AMP_BWD writes it
        assert rel_max(host(t["db"]), db_ref) < 1e-4
    finally:
        plugin.trbh_destroy(hnd)


def test_grad_scaling_and_single_rank_allreduce_nodes(plugin):
    """RANGE_GRAD_SCALING through g_range_op_table, and RANGE_MEAN_ALLREDUCE with one rank (a no-op that still keeps
    the stream protocol, allreduce_op.cpp:47-51)."""
    _range_api(plugin)
    flag = torch.ones(1, dtype=torch.int32, device="cuda")
    scaling = torch.tensor([1024.0], device="cuda")
    arena = torch.arange(1024, dtype=torch.float32, device="cuda")
    hnd = plugin.trbh_create()
    try:
        _ok(plugin, plugin.trbh_set_rank(hnd, 0, 1, arena.data_ptr()))
        _add(plugin, hnd, 1, flag, (1, 1, 1, 1), INT32)
        _add(plugin, hnd, 2, scaling, (1, 1, 1, 1), FP32)
        ids, n_ids = _ids([1, 2])
        _ok(plugin, plugin.trbh_add_range_node(hnd, R_GRAD_SCALING, 0, 0, 0, ids, n_ids))
        _ok(plugin, plugin.trbh_add_range_node(hnd, R_MEAN_AR, 7, 256, 512, None, 0))
        _ok(plugin, plugin.trbh_warmup(hnd))
        assert float(scaling) == 512.0
        _ok(plugin, plugin.trbh_capture(hnd))
        _ok(plugin, plugin.trbh_replay(hnd))
        assert float(scaling) == 256.0
        assert torch.equal(arena, torch.arange(1024, dtype=torch.float32, device="cuda"))
    finally:
        plugin.trbh_destroy(hnd)


def _allreduce_rank(rank, world, id_path, out_path):
    """One rank of the two-GPU all-reduce test (a child process: one NCCL communicator per process)."""
    import time
    torch.cuda.set_device(rank)
    from renaissance_b200 import _lib
    _lib.load()
    lib = _range_api(C.CDLL(os.path.join(os.path.dirname(_lib.LIB_PATH), "libtrb200_plugin.so")))
    lib.trbh_create.restype = C.c_void_p
    lib.trbh_last_error.restype = C.c_char_p
    lib.trbh_destroy.argtypes = [C.c_void_p]
    for f in (lib.trbh_warmup, lib.trbh_capture, lib.trbh_replay):
        f.argtypes = [C.c_void_p]
    uid = C.create_string_buffer(128)
    if rank == 0:
        assert lib.trbh_nccl_unique_id(uid) == 0, lib.trbh_last_error()
        with open(id_path + ".tmp", "wb") as fh:
            fh.write(uid.raw)
        os.replace(id_path + ".tmp", id_path)
    else:
        for _ in range(600):
            if os.path.exists(id_path):
                break
            time.sleep(0.05)
        with open(id_path, "rb") as fh:
            uid = C.create_string_buffer(fh.read(), 128)
    hnd = lib.trbh_create()
    assert lib.trbh_nccl_init(hnd, world, rank, uid) == 0, lib.trbh_last_error()
    n = 1 << 20
    arena = torch.full((n,), float(rank + 1), device="cuda")
    arena[7] = 100.0 * (rank + 1)
    assert lib.trbh_set_rank(hnd, rank, world, arena.data_ptr()) == 0
    # two spans: a mean over [0, n/2) and a sum over [n/2, n)
    assert lib.trbh_add_range_node(hnd, R_MEAN_AR, 3, 0, n // 2 * 4, None, 0) == 0
    assert lib.trbh_add_range_node(hnd, R_SUM_AR, 4, n // 2 * 4, n // 2 * 4, None, 0) == 0
    assert lib.trbh_warmup(hnd) == 0, lib.trbh_last_error()
    torch.cuda.synchronize()
    res = arena.cpu().numpy().copy()
    lib.trbh_nccl_destroy(hnd)
    lib.trbh_destroy(hnd)
    np.save(out_path, res)


def test_mean_allreduce_launcher_on_two_gpus(tmp_path):
    """RANGE_MEAN_ALLREDUCE / RANGE_SUM_ALLREDUCE through the registry on two GPUs (one process each, NCCL over
    NVLink, NVLS off): every rank ends with the same values, the mean of the ranks' on one span and the sum on the
    other (the reference's test_mean_allreduce.cpp:96-136 checks the same)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import subprocess
    import sys
    id_path = str(tmp_path / "nccl_id.bin")
    outs = [str(tmp_path / f"rank{r}.npy") for r in range(2)]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    code = ("import sys; sys.path.insert(0, {root!r}); sys.path.insert(0, {tests!r}); "
            "import test_gpu_plugin_registry as t; t._allreduce_rank({rank}, 2, {idp!r}, {out!r})")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    procs = [subprocess.Popen([sys.executable, "-c", code.format(root=root, tests=os.path.join(root, "tests"), rank=r,
                                                                  idp=id_path, out=outs[r])], env=env)
             for r in range(2)]
    for p in procs:
        assert p.wait(timeout=120) == 0
    a, b = np.load(outs[0]), np.load(outs[1])
    assert np.array_equal(a, b)                                   # identical on both ranks
    n = a.size
    assert np.all(a[:7] == 1.5) and a[7] == 150.0 and np.all(a[8:n // 2] == 1.5)      # mean of 1 and 2
    assert np.all(a[n // 2:] == 3.0)                                                  # sum
