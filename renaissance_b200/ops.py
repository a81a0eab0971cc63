"""Host-side mirror of the reference launchers for the hot path.

Each function takes torch CUDA tensors (device memory and streams are torch's;
all arithmetic is in libtrb200.so), checks shapes the way the reference
launcher derives them from its DTensors, and makes ONE C-ABI call.

    cbr_amp_bwd            launch_cbr_amp_bwd_cuda             cbr_op.cpp:1359-1522
    cbr_amp_bwd(dx=None)   launch_cbr_amp_bwd_first_layer_cuda cbr_op.cpp:1528-1651
    softmax_ce_amp_fwd     launch_softmax_ce_amp_fwd_cuda      softmax_ce_op.cpp:409-455
    softmax_ce_amp_bwd     launch_softmax_ce_amp_bwd_cuda      softmax_ce_op.cpp:591-627
    softmax_ce_amp_fused   both nodes in one kernel
    mean_allreduce         launch_allreduce_cuda_impl          allreduce_op.cpp:37-105
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import CbrBwdArgs, ConvDesc, check


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream(stream=None):
    s = torch.cuda.current_stream() if stream is None else stream
    return C.c_void_p(s.cuda_stream)


# TRB200_DTYPE_* of include/trb200.h
DTYPE_CODE = {torch.float16: 0, torch.bfloat16: 1}


def _need(t, dtype, name, ndim=None):
    if not (isinstance(t, torch.Tensor) and t.is_cuda):
        raise TypeError(f"{name}: CUDA tensor expected")
    if t.dtype != dtype:
        raise TypeError(f"{name}: dtype {dtype} expected, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name}: compact (contiguous) tensor expected")
    if ndim is not None and t.dim() != ndim:
        raise ValueError(f"{name}: {ndim} dimensions expected, got {tuple(t.shape)}")


@dataclass
class ConvGeometry:
    """ConvParams of the reference (include/renaissance/graph/op_kind.h:42-52)."""
    n: int
    h: int
    w: int
    c: int
    k: int
    r: int = 3
    s: int = 3
    pad: int = 1
    stride: int = 1
    dtype: torch.dtype = torch.float16     # storage type of activations, filters and their gradients

    def desc(self) -> ConvDesc:
        return ConvDesc(self.n, self.h, self.w, self.c, self.k, self.r, self.s,
                        self.pad, self.pad, self.stride, self.stride, DTYPE_CODE[self.dtype])

    @property
    def oh(self):
        return (self.h + 2 * self.pad - self.r) // self.stride + 1

    @property
    def ow(self):
        return (self.w + 2 * self.pad - self.s) // self.stride + 1


class Workspace:
    """Grow-only device scratch, the DeviceContext::ensure_workspace_grow contract
    (src/backend/device_context.cpp:379-428): sized in the warm-up call, reused after."""

    def __init__(self, device=None):
        self.device = device
        self.buf = None

    def ensure(self, nbytes: int) -> torch.Tensor:
        nbytes = max(int(nbytes), 256)
        if self.buf is None or self.buf.numel() < nbytes:
            self.buf = torch.empty(nbytes, dtype=torch.uint8, device=self.device or "cuda")
        return self.buf


_default_ws: dict[int, Workspace] = {}


def default_workspace() -> Workspace:
    dev = torch.cuda.current_device()
    if dev not in _default_ws:
        _default_ws[dev] = Workspace(torch.device("cuda", dev))
    return _default_ws[dev]


def kernel_launch_count() -> int:
    """Kernels launched by libtrb200.so in this process so far."""
    return int(_lib.load().trb200_kernel_launch_count())


def device_status() -> None:
    """Synchronise, then raise if any kernel's bounded device-side wait gave up."""
    torch.cuda.synchronize()
    check(_lib.load().trb200_device_status())


def selftest_wait_timeout(limit_ns: int = 1_000_000, stream=None):
    """Runs the library's bounded wait on a barrier nobody arrives on.  Returns a 4-int device tensor
    {warp 0 got it, ns waited, warp 1 got it, ns waited}; device_status() raises afterwards (once)."""
    out = torch.zeros(4, dtype=torch.int32, device="cuda")
    check(_lib.load().trb200_selftest_wait_timeout(int(limit_ns), _ptr(out), _stream(stream)))
    return out


def set_conv_backend(direct_only: bool) -> None:
    check(_lib.load().trb200_set_conv_backend(1 if direct_only else 0))


def conv_uses_tensor_cores(g: ConvGeometry, which: str) -> bool:
    idx = {"wgrad": 0, "dgrad": 1, "fprop": 2}[which]
    d = g.desc()
    return bool(_lib.load().trb200_conv_uses_tensor_cores(C.byref(d), idx))


# --------------------------------------------------------------------------- BN + ReLU backward

def bnrelu_bwd(dy, mask_bits, conv_out, gamma, saved_mean, saved_inv_std, dconv=None,
               workspace: Workspace | None = None, stream=None, want_dconv=True):
    """dconv, dgamma, dbeta of the block's BN+ReLU (cbr_op.cpp:1259-1353).  mask_bits=None: a BN with no ReLU
    behind it (plain batch-norm backward)."""
    lib = _lib.load()
    if dy.dtype not in DTYPE_CODE:
        raise TypeError(f"dy: float16 or bfloat16 expected, got {dy.dtype}")
    _need(dy, dy.dtype, "dy")
    _need(conv_out, dy.dtype, "conv_out")
    if mask_bits is not None:
        _need(mask_bits, torch.uint8, "mask_bits")
    for t, nm in ((gamma, "gamma"), (saved_mean, "saved_mean"), (saved_inv_std, "saved_inv_std")):
        _need(t, torch.float32, nm)
    c = dy.shape[-1]
    m = dy.numel() // c
    if conv_out.shape != dy.shape:
        raise ValueError("conv_out and dy must have the same shape")
    if mask_bits is not None and mask_bits.numel() * 8 < dy.numel():
        raise ValueError("mask_bits holds fewer bits than dy has elements")
    if dconv is None and want_dconv:
        dconv = torch.empty_like(dy)
    dgamma = torch.empty(c, dtype=torch.float32, device=dy.device)
    dbeta = torch.empty(c, dtype=torch.float32, device=dy.device)
    ws = (workspace or default_workspace()).ensure(lib.trb200_bnrelu_bwd_workspace_bytes(m, c))
    check(lib.trb200_bnrelu_bwd_dtype(_ptr(dy), _ptr(mask_bits), _ptr(conv_out), _ptr(gamma), _ptr(saved_mean),
                                      _ptr(saved_inv_std), _ptr(dconv), _ptr(dgamma), _ptr(dbeta), m, c,
                                      DTYPE_CODE[dy.dtype], _ptr(ws), ws.numel(), _stream(stream)))
    return dconv, dgamma, dbeta


# --------------------------------------------------------------------------- general pooling

def maxpool_fwd(x, k=3, stride=2, pad=1, stream=None):
    """k x k max pool; returns (y, argmax byte per element)."""
    _need(x, x.dtype, "x", 4)
    n, h, w, c = x.shape
    oh, ow = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
    y = torch.empty((n, oh, ow, c), dtype=x.dtype, device=x.device)
    am = torch.empty((n, oh, ow, c), dtype=torch.uint8, device=x.device)
    check(_lib.load().trb200_maxpool_fwd(_ptr(x), _ptr(y), _ptr(am), n, h, w, c, k, stride, pad, DTYPE_CODE[x.dtype],
                                         _stream(stream)))
    return y, am


def maxpool_bwd(dy, argmax, x_shape, k=3, stride=2, pad=1, stream=None):
    _need(dy, dy.dtype, "dy", 4)
    _need(argmax, torch.uint8, "argmax", 4)
    n, h, w, c = x_shape
    dx = torch.empty((n, h, w, c), dtype=dy.dtype, device=dy.device)
    check(_lib.load().trb200_maxpool_bwd(_ptr(dy), _ptr(argmax), _ptr(dx), n, h, w, c, k, stride, pad,
                                         DTYPE_CODE[dy.dtype], _stream(stream)))
    return dx


def avgpool_global_fwd(x, stream=None):
    _need(x, x.dtype, "x", 4)
    n, h, w, c = x.shape
    y = torch.empty((n, c), dtype=x.dtype, device=x.device)
    check(_lib.load().trb200_avgpool_global_fwd(_ptr(x), _ptr(y), n, h, w, c, DTYPE_CODE[x.dtype], _stream(stream)))
    return y


def avgpool_global_bwd(dy, h, w, stream=None):
    _need(dy, dy.dtype, "dy", 2)
    n, c = dy.shape
    dx = torch.empty((n, h, w, c), dtype=dy.dtype, device=dy.device)
    check(_lib.load().trb200_avgpool_global_bwd(_ptr(dy), _ptr(dx), n, h, w, c, DTYPE_CODE[dy.dtype], _stream(stream)))
    return dx


# --------------------------------------------------------------------------- residual join

def add16(a, b, out=None, stream=None):
    """out = a + b in the tensors' 16-bit type (join of two branches or of their gradients)."""
    _need(a, a.dtype, "a")
    _need(b, a.dtype, "b")
    out = torch.empty_like(a) if out is None else out
    check(_lib.load().trb200_add16(_ptr(a), _ptr(b), _ptr(out), a.numel(), DTYPE_CODE[a.dtype], _stream(stream)))
    return out


def add_relu_mask(a, b, out=None, mask_bits=None, stream=None):
    """relu(a + b) and its bit-packed mask: the end of a residual block."""
    _need(a, a.dtype, "a")
    _need(b, a.dtype, "b")
    out = torch.empty_like(a) if out is None else out
    if mask_bits is None:
        mask_bits = torch.empty(a.numel() // 8, dtype=torch.uint8, device=a.device)
    check(_lib.load().trb200_add_relu_mask(_ptr(a), _ptr(b), _ptr(out), _ptr(mask_bits), a.numel(),
                                           DTYPE_CODE[a.dtype], _stream(stream)))
    return out, mask_bits


def relu_mask_bwd(dy, mask_bits, dx=None, stream=None):
    """dx = mask ? dy : 0 with the block's bit-packed mask."""
    _need(dy, dy.dtype, "dy")
    _need(mask_bits, torch.uint8, "mask_bits")
    dx = torch.empty_like(dy) if dx is None else dx
    check(_lib.load().trb200_relu_mask_bwd(_ptr(dy), _ptr(mask_bits), _ptr(dx), dy.numel(), _stream(stream)))
    return dx


# --------------------------------------------------------------------------- conv gradients

def conv_wgrad(g: ConvGeometry, dy, x, dw=None, workspace=None, stream=None):
    lib = _lib.load()
    _need(dy, g.dtype, "dy", 4)
    _need(x, g.dtype, "x", 4)
    if tuple(x.shape) != (g.n, g.h, g.w, g.c) or tuple(dy.shape) != (g.n, g.oh, g.ow, g.k):
        raise ValueError("conv_wgrad: tensor shapes do not match the geometry")
    if dw is None:
        dw = torch.empty((g.k, g.r, g.s, g.c), dtype=g.dtype, device=x.device)
    d = g.desc()
    ws = (workspace or default_workspace()).ensure(lib.trb200_conv_wgrad_workspace_bytes(C.byref(d)))
    check(lib.trb200_conv_wgrad(C.byref(d), _ptr(dy), _ptr(x), _ptr(dw), _ptr(ws), ws.numel(), _stream(stream)))
    return dw


def conv_dgrad(g: ConvGeometry, dy, w, dx=None, workspace=None, stream=None):
    lib = _lib.load()
    _need(dy, g.dtype, "dy", 4)
    _need(w, g.dtype, "w", 4)
    if tuple(w.shape) != (g.k, g.r, g.s, g.c) or tuple(dy.shape) != (g.n, g.oh, g.ow, g.k):
        raise ValueError("conv_dgrad: tensor shapes do not match the geometry")
    if dx is None:
        dx = torch.empty((g.n, g.h, g.w, g.c), dtype=g.dtype, device=dy.device)
    d = g.desc()
    ws = (workspace or default_workspace()).ensure(lib.trb200_conv_dgrad_workspace_bytes(C.byref(d)))
    check(lib.trb200_conv_dgrad(C.byref(d), _ptr(dy), _ptr(w), _ptr(dx), _ptr(ws), ws.numel(), _stream(stream)))
    return dx


def conv_fprop(g: ConvGeometry, x, w, y=None, stream=None, workspace=None, scratch=None):
    lib = _lib.load()
    _need(x, g.dtype, "x", 4)
    _need(w, g.dtype, "w", 4)
    if tuple(x.shape) != (g.n, g.h, g.w, g.c) or tuple(w.shape) != (g.k, g.r, g.s, g.c):
        raise ValueError("conv_fprop: tensor shapes do not match the geometry")
    if y is None:
        y = torch.empty((g.n, g.oh, g.ow, g.k), dtype=g.dtype, device=x.device)
    d = g.desc()
    need = lib.trb200_conv_fprop_workspace_bytes(C.byref(d))
    if scratch is not None and scratch.numel() * scratch.element_size() >= need:
        ws, ws_bytes = scratch, scratch.numel() * scratch.element_size()     # caller's free activation buffer
    else:
        ws = (workspace or default_workspace()).ensure(need)
        ws_bytes = ws.numel()
    check(lib.trb200_conv_fprop(C.byref(d), _ptr(x), _ptr(w), _ptr(y), _ptr(ws), ws_bytes, _stream(stream)))
    return y


def conv_fprop_bn_stats(g: ConvGeometry, x, w, gamma, beta, y=None, out=None, eps=1e-5, momentum=0.1,
                        running_mean=None, running_var=None, workspace=None, scratch=None, stream=None,
                        want_sums=False):
    """Forward conv + batch statistics in its epilogue + bn_finalize (cbr_op.cpp:622-718, 430-528).
    Returns (y, dict(saved_mean, saved_inv_std, eq_scale, eq_bias[, sum, sqsum]))."""
    lib = _lib.load()
    _need(x, g.dtype, "x", 4)
    _need(w, g.dtype, "w", 4)
    if tuple(x.shape) != (g.n, g.h, g.w, g.c) or tuple(w.shape) != (g.k, g.r, g.s, g.c):
        raise ValueError("conv_fprop_bn_stats: tensor shapes do not match the geometry")
    dev = x.device
    if y is None:
        y = torch.empty((g.n, g.oh, g.ow, g.k), dtype=g.dtype, device=dev)
    if out is None:
        out = {k: torch.empty(g.k, dtype=torch.float32, device=dev)
               for k in ("saved_mean", "saved_inv_std", "eq_scale", "eq_bias")}
    if want_sums:
        out["sum"] = torch.empty(g.k, dtype=torch.float32, device=dev)
        out["sqsum"] = torch.empty(g.k, dtype=torch.float32, device=dev)
    d = g.desc()
    need = lib.trb200_conv_fprop_bn_stats_workspace_bytes(C.byref(d))
    if scratch is not None and scratch.numel() * scratch.element_size() >= need:
        ws, ws_bytes = scratch, scratch.numel() * scratch.element_size()
    else:
        ws = (workspace or default_workspace()).ensure(need)
        ws_bytes = ws.numel()
    check(lib.trb200_conv_fprop_bn_stats(C.byref(d), _ptr(x), _ptr(w), _ptr(y), _ptr(gamma), _ptr(beta), float(eps),
                                         float(momentum), _ptr(out.get("sum")), _ptr(out.get("sqsum")),
                                         _ptr(out["saved_mean"]), _ptr(out["saved_inv_std"]), _ptr(out["eq_scale"]),
                                         _ptr(out["eq_bias"]), _ptr(running_mean), _ptr(running_var), _ptr(ws),
                                         ws_bytes, _stream(stream)))
    return y, out


# --------------------------------------------------------------------------- whole block

@dataclass
class BlockStreams:
    """The three compute streams of the reference's DeviceContext and the per-stream
    `last_done_event`s of its MultiStreamCaptureState (capture_multi_stream.h:25-46)."""
    bn: torch.cuda.Stream
    wgrad: torch.cuda.Stream
    dgrad: torch.cuda.Stream
    ev_bn: torch.cuda.Event
    ev_wgrad: torch.cuda.Event
    ev_dgrad: torch.cuda.Event

    @staticmethod
    def create(device=None) -> "BlockStreams":
        mk = lambda: torch.cuda.Stream(device=device)
        ev = lambda: torch.cuda.Event(enable_timing=False)
        out = BlockStreams(mk(), mk(), mk(), ev(), ev(), ev())
        # torch creates the underlying cudaEvent lazily: record once so that the handle exists
        for e, s in ((out.ev_bn, out.bn), (out.ev_wgrad, out.wgrad), (out.ev_dgrad, out.dgrad)):
            e.record(s)
        return out


def cbr_amp_bwd(g: ConvGeometry, dy, w, gamma, saved_mean, saved_inv_std, mask_bits, x, conv_out,
                bn_scratch=None, dw=None, first_layer=False, streams: BlockStreams | None = None,
                workspace=None, stream=None, dgamma=None, dbeta=None, pool_argmax=None, timing_events=None):
    """CBR_AMP_BWD / CBR_AMP_BWD_FIRST_LAYER.

    Node ids of the reference: in [dY, W16, gamma, saved_mean, saved_inv_var, mask, X],
    out [dX (= X's buffer), dW16, dgamma, dbeta, conv_output, bn_output]
    (cbr_op.cpp:1365-1366).  As there, dX is written IN PLACE over ``x`` (returned as
    ``dx``) unless ``first_layer``.  With ``pool_argmax`` the block is followed by a 2x2 max pool and
    ``dy`` is the gradient of the pooled output.  Returns dict(dx, dw, dgamma, dbeta, dconv)."""
    lib = _lib.load()
    _need(dy, g.dtype, "dy", 4)
    _need(w, g.dtype, "w", 4)
    _need(x, g.dtype, "x", 4)
    _need(conv_out, g.dtype, "conv_out", 4)
    _need(mask_bits, torch.uint8, "mask_bits")
    for t, nm in ((gamma, "gamma"), (saved_mean, "saved_mean"), (saved_inv_std, "saved_inv_std")):
        _need(t, torch.float32, nm)
    dy_shape = (g.n, g.oh, g.ow, g.k) if pool_argmax is None else (g.n, g.oh // 2, g.ow // 2, g.k)
    if tuple(x.shape) != (g.n, g.h, g.w, g.c) or tuple(dy.shape) != dy_shape \
            or tuple(w.shape) != (g.k, g.r, g.s, g.c) or tuple(conv_out.shape) != (g.n, g.oh, g.ow, g.k):
        raise ValueError("cbr_amp_bwd: tensor shapes do not match the geometry")
    if bn_scratch is None:
        bn_scratch = torch.empty_like(conv_out)
    if dw is None:
        dw = torch.empty_like(w)
    if dgamma is None:
        dgamma = torch.empty(g.k, dtype=torch.float32, device=x.device)
    if dbeta is None:
        dbeta = torch.empty(g.k, dtype=torch.float32, device=x.device)
    d = g.desc()
    ws = (workspace or default_workspace()).ensure(lib.trb200_cbr_bwd_workspace_bytes(C.byref(d), int(first_layer)))
    a = CbrBwdArgs()
    a.conv = d
    a.dy, a.w, a.gamma = dy.data_ptr(), w.data_ptr(), gamma.data_ptr()
    a.saved_mean, a.saved_inv_std = saved_mean.data_ptr(), saved_inv_std.data_ptr()
    a.mask_bits, a.x = mask_bits.data_ptr(), x.data_ptr()
    a.dx = None if first_layer else x.data_ptr()
    a.dw, a.dgamma, a.dbeta = dw.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr()
    a.conv_out, a.bn_scratch = conv_out.data_ptr(), bn_scratch.data_ptr()
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    a.pool_argmax = None if pool_argmax is None else pool_argmax.data_ptr()
    if streams is None:
        s = (torch.cuda.current_stream() if stream is None else stream).cuda_stream
        a.stream_bn = a.stream_wgrad = a.stream_dgrad = s
        a.ev_bn = a.ev_wgrad = a.ev_dgrad = None
    else:
        a.stream_bn, a.stream_wgrad, a.stream_dgrad = (streams.bn.cuda_stream, streams.wgrad.cuda_stream,
                                                      streams.dgrad.cuda_stream)
        a.ev_bn, a.ev_wgrad, a.ev_dgrad = (streams.ev_bn.cuda_event, streams.ev_wgrad.cuda_event,
                                           streams.ev_dgrad.cuda_event)
    if timing_events is not None:        # four torch events (enable_timing=True): start, after BN, wgrad, dgrad
        for i, ev in enumerate(timing_events):
            if ev is not None and not (first_layer and i == 3):
                ev.record(torch.cuda.current_stream())      # creates the handle; re-recorded inside the call
                a.ev_time[i] = ev.cuda_event
    check(lib.trb200_cbr_bwd(C.byref(a)))
    return dict(dx=None if first_layer else x, dw=dw, dgamma=dgamma, dbeta=dbeta, dconv=bn_scratch)


# --------------------------------------------------------------------------- forward side of the block

def bn_stats_finalize(conv_out, gamma, beta, eps=1e-5, momentum=0.1, running_mean=None, running_var=None,
                      out=None, workspace=None, stream=None, want_sums=False):
    """Batch statistics of the conv output + bn_finalize (cbr_op.cpp:430-528, 622-718).
    Returns dict(saved_mean, saved_inv_std, eq_scale, eq_bias[, sum, sqsum])."""
    lib = _lib.load()
    if conv_out.dtype not in DTYPE_CODE:
        raise TypeError(f"conv_out: float16 or bfloat16 expected, got {conv_out.dtype}")
    _need(conv_out, conv_out.dtype, "conv_out")
    c = conv_out.shape[-1]
    m = conv_out.numel() // c
    dev = conv_out.device
    if out is None:
        out = {k: torch.empty(c, dtype=torch.float32, device=dev)
               for k in ("saved_mean", "saved_inv_std", "eq_scale", "eq_bias")}
    if want_sums:
        out["sum"] = torch.empty(c, dtype=torch.float32, device=dev)
        out["sqsum"] = torch.empty(c, dtype=torch.float32, device=dev)
    ws = (workspace or default_workspace()).ensure(lib.trb200_bn_stats_workspace_bytes(m, c))
    check(lib.trb200_bn_stats_finalize_dtype(_ptr(conv_out), _ptr(gamma), _ptr(beta), float(eps), float(momentum),
                                             _ptr(out.get("sum")), _ptr(out.get("sqsum")), _ptr(out["saved_mean"]),
                                             _ptr(out["saved_inv_std"]), _ptr(out["eq_scale"]), _ptr(out["eq_bias"]),
                                             _ptr(running_mean), _ptr(running_var), m, c, DTYPE_CODE[conv_out.dtype],
                                             _ptr(ws), ws.numel(), _stream(stream)))
    return out


def bn_apply(conv_out, eq_scale, eq_bias, relu=True, out=None, mask_bits=None, stream=None):
    """The apply stage for half or bfloat16 tensors: with relu, (relu_out, bit-packed mask) as bn_apply_relu_mask;
    without, (bn_out, None): the BN in front of a residual join."""
    if conv_out.dtype not in DTYPE_CODE:
        raise TypeError(f"conv_out: float16 or bfloat16 expected, got {conv_out.dtype}")
    _need(conv_out, conv_out.dtype, "conv_out")
    c = conv_out.shape[-1]
    m = conv_out.numel() // c
    if out is None:
        out = torch.empty_like(conv_out)
    if relu and mask_bits is None:
        mask_bits = torch.empty(conv_out.numel() // 8, dtype=torch.uint8, device=conv_out.device)
    check(_lib.load().trb200_bn_apply_dtype(_ptr(conv_out), _ptr(eq_scale), _ptr(eq_bias), _ptr(out),
                                            _ptr(mask_bits) if relu else None, m, c, 1 if relu else 0,
                                            DTYPE_CODE[conv_out.dtype], _stream(stream)))
    return out, (mask_bits if relu else None)


def bn_apply_relu_mask(conv_out, eq_scale, eq_bias, relu_out=None, mask_bits=None, stream=None):
    """relu_out and the bit-packed ReLU mask (cbr_op.cpp:534-616)."""
    lib = _lib.load()
    _need(conv_out, torch.float16, "conv_out")
    c = conv_out.shape[-1]
    m = conv_out.numel() // c
    if relu_out is None:
        relu_out = torch.empty_like(conv_out)
    if mask_bits is None:
        mask_bits = torch.empty(conv_out.numel() // 8, dtype=torch.uint8, device=conv_out.device)
    check(lib.trb200_bn_apply_relu_mask(_ptr(conv_out), _ptr(eq_scale), _ptr(eq_bias), _ptr(relu_out),
                                        _ptr(mask_bits), m, c, _stream(stream)))
    return relu_out, mask_bits


def bn_apply_relu_mask_pool(conv_out, eq_scale, eq_bias, mask_bits=None, pool_out=None, argmax=None, relu_out=None,
                            stream=None):
    """BN apply + ReLU + mask + 2x2 max pool in one kernel; relu_out is written only if given."""
    _need(conv_out, torch.float16, "conv_out", 4)
    n, h, w, c = conv_out.shape
    dev = conv_out.device
    if mask_bits is None:
        mask_bits = torch.empty(conv_out.numel() // 8, dtype=torch.uint8, device=dev)
    if pool_out is None:
        pool_out = torch.empty((n, h // 2, w // 2, c), dtype=torch.float16, device=dev)
    if argmax is None:
        argmax = torch.empty((n, h // 2, w // 2, c), dtype=torch.uint8, device=dev)
    check(_lib.load().trb200_bn_apply_relu_mask_pool(_ptr(conv_out), _ptr(eq_scale), _ptr(eq_bias), _ptr(relu_out),
                                                     _ptr(mask_bits), _ptr(pool_out), _ptr(argmax), n, h, w, c,
                                                     _stream(stream)))
    return pool_out, argmax, mask_bits


def bnrelu_pool_bwd(dy_pooled, argmax, mask_bits, conv_out, gamma, saved_mean, saved_inv_std, dconv=None,
                    workspace=None, stream=None):
    """max-pool backward + BN/ReLU backward of the block in one pair of sweeps."""
    lib = _lib.load()
    _need(dy_pooled, torch.float16, "dy_pooled", 4)
    _need(conv_out, torch.float16, "conv_out", 4)
    n, h, w, c = conv_out.shape
    if tuple(dy_pooled.shape) != (n, h // 2, w // 2, c):
        raise ValueError("bnrelu_pool_bwd: dy_pooled must be [n, h/2, w/2, c]")
    if dconv is None:
        dconv = torch.empty_like(conv_out)
    dgamma = torch.empty(c, dtype=torch.float32, device=conv_out.device)
    dbeta = torch.empty(c, dtype=torch.float32, device=conv_out.device)
    ws = (workspace or default_workspace()).ensure(lib.trb200_bnrelu_pool_bwd_workspace_bytes(n, h, w, c))
    check(lib.trb200_bnrelu_pool_bwd(_ptr(dy_pooled), _ptr(argmax), _ptr(mask_bits), _ptr(conv_out), _ptr(gamma),
                                     _ptr(saved_mean), _ptr(saved_inv_std), _ptr(dconv), _ptr(dgamma), _ptr(dbeta),
                                     n, h, w, c, _ptr(ws), ws.numel(), _stream(stream)))
    return dconv, dgamma, dbeta


def maxpool2x2_fwd(x, y=None, argmax=None, stream=None):
    _need(x, torch.float16, "x", 4)
    n, h, w, c = x.shape
    if y is None:
        y = torch.empty((n, h // 2, w // 2, c), dtype=torch.float16, device=x.device)
    if argmax is None:
        argmax = torch.empty((n, h // 2, w // 2, c), dtype=torch.uint8, device=x.device)
    check(_lib.load().trb200_maxpool2x2_fwd(_ptr(x), _ptr(y), _ptr(argmax), n, h, w, c, _stream(stream)))
    return y, argmax


def maxpool2x2_bwd(dy, argmax, dx, stream=None):
    _need(dy, torch.float16, "dy", 4)
    n, h, w, c = dx.shape
    check(_lib.load().trb200_maxpool2x2_bwd(_ptr(dy), _ptr(argmax), _ptr(dx), n, h, w, c, _stream(stream)))
    return dx


def check_nonfinite(flat_f32, flag, stream=None):
    check(_lib.load().trb200_check_nonfinite(_ptr(flat_f32), flat_f32.numel(), _ptr(flag), _stream(stream)))


def sgd_momentum(w32, g32, m32, w16, lr, weight_decay, beta, scaling=None, skip_flag=None, stream=None):
    check(_lib.load().trb200_sgd_momentum(_ptr(w32), _ptr(g32), _ptr(m32), _ptr(w16), w32.numel(), float(lr),
                                          float(weight_decay), float(beta), _ptr(scaling), _ptr(skip_flag),
                                          _stream(stream)))


def sgd_nesterov(w32, g32, m32, w16, lr, weight_decay, beta, scaling=None, skip_flag=None, stream=None):
    check(_lib.load().trb200_sgd_nesterov(_ptr(w32), _ptr(g32), _ptr(m32), _ptr(w16), w32.numel(), float(lr),
                                          float(weight_decay), float(beta), _ptr(scaling), _ptr(skip_flag),
                                          _stream(stream)))


def sgd_plain(w32, g32, w16, lr, weight_decay, scaling=None, skip_flag=None, stream=None):
    check(_lib.load().trb200_sgd_plain(_ptr(w32), _ptr(g32), _ptr(w16), w32.numel(), float(lr), float(weight_decay),
                                       _ptr(scaling), _ptr(skip_flag), _stream(stream)))


def check_nan_and_clip(flat_f32, clip, flag, stream=None):
    check(_lib.load().trb200_check_nan_and_clip(_ptr(flat_f32), flat_f32.numel(), float(clip), _ptr(flag), _stream(stream)))


def grad_scaling(flag, scaling, clear_flag=False, stream=None):
    """Loss-scale back-off: halves `scaling` (never below 1) if `flag` is set; optionally resets the flag."""
    check(_lib.load().trb200_grad_scaling(_ptr(flag), _ptr(scaling), 1 if clear_flag else 0, _stream(stream)))


# --------------------------------------------------------------------------- softmax + CE

def softmax_ce_amp_fwd(logits, labels, label_smoothing, probs=None, want_probs=True, stream=None):
    """SOFTMAX_CE_AMP_FWD: returns dict(loss, inv_scaling, probs, loss_partial) (device tensors)."""
    lib = _lib.load()
    _need(logits, torch.float16, "logits", 2)
    _need(labels, torch.int32, "labels", 1)
    _need(label_smoothing, torch.float32, "label_smoothing")
    b, k = logits.shape
    dev = logits.device
    if probs is None and want_probs:
        probs = torch.empty((b, k), dtype=torch.float32, device=dev)
    part = torch.empty(b, dtype=torch.float32, device=dev)
    loss = torch.empty(1, dtype=torch.float32, device=dev)
    inv = torch.empty(1, dtype=torch.float32, device=dev)
    check(lib.trb200_softmax_ce_fwd(_ptr(logits), logits.stride(0), _ptr(labels), _ptr(label_smoothing),
                                    _ptr(probs), 0 if probs is None else probs.stride(0),
                                    _ptr(part), _ptr(loss), _ptr(inv), b, k, _stream(stream)))
    return dict(loss=loss, inv_scaling=inv, probs=probs, loss_partial=part)


def softmax_ce_amp_bwd(probs, labels, scaling, inv_scaling, label_smoothing, dlogits=None, stream=None):
    """SOFTMAX_CE_AMP_BWD: d_logits half [B, C]."""
    lib = _lib.load()
    _need(probs, torch.float32, "probs", 2)
    _need(labels, torch.int32, "labels", 1)
    b, k = probs.shape
    if dlogits is None:
        dlogits = torch.empty((b, k), dtype=torch.float16, device=probs.device)
    check(lib.trb200_softmax_ce_bwd(_ptr(probs), probs.stride(0), _ptr(labels), _ptr(scaling), _ptr(inv_scaling),
                                    _ptr(label_smoothing), _ptr(dlogits), dlogits.stride(0), b, k, _stream(stream)))
    return dlogits


def softmax_ce_amp_fused(logits, labels, scaling, label_smoothing, want_probs=False, dlogits=None, stream=None):
    """FWD + BWD nodes in one pass over the logits.  bfloat16 logits: without probs, at most 2048 classes."""
    lib = _lib.load()
    if logits.dtype not in DTYPE_CODE:
        raise TypeError(f"logits: float16 or bfloat16 expected, got {logits.dtype}")
    if not (isinstance(logits, torch.Tensor) and logits.is_cuda and logits.dim() == 2 and logits.stride(1) == 1):
        raise ValueError("logits: a 2-D CUDA tensor with unit column stride expected (rows may be padded)")
    if dlogits is not None and not (dlogits.dim() == 2 and dlogits.stride(1) == 1 and dlogits.dtype == logits.dtype):
        raise ValueError("dlogits: a 2-D tensor of the logits' type with unit column stride expected")
    _need(labels, torch.int32, "labels", 1)
    b, k = logits.shape
    dev = logits.device
    probs = torch.empty((b, k), dtype=torch.float32, device=dev) if want_probs else None
    if dlogits is None:
        dlogits = torch.empty((b, k), dtype=logits.dtype, device=dev)
    part = torch.empty(b, dtype=torch.float32, device=dev)
    loss = torch.empty(1, dtype=torch.float32, device=dev)
    inv = torch.empty(1, dtype=torch.float32, device=dev)
    if logits.dtype == torch.bfloat16:
        if want_probs:
            raise ValueError("softmax_ce_amp_fused: bfloat16 logits are supported without probs only")
        check(lib.trb200_softmax_ce_fused_dtype(_ptr(logits), logits.stride(0), _ptr(labels), _ptr(scaling),
                                                _ptr(label_smoothing), _ptr(dlogits), dlogits.stride(0), _ptr(part),
                                                _ptr(loss), _ptr(inv), b, k, DTYPE_CODE[logits.dtype],
                                                _stream(stream)))
        return dict(loss=loss, inv_scaling=inv, probs=None, loss_partial=part, dlogits=dlogits)
    check(lib.trb200_softmax_ce_fused(_ptr(logits), logits.stride(0), _ptr(labels), _ptr(scaling),
                                      _ptr(label_smoothing), _ptr(probs), 0 if probs is None else probs.stride(0),
                                      _ptr(dlogits), dlogits.stride(0), _ptr(part), _ptr(loss), _ptr(inv),
                                      b, k, _stream(stream)))
    return dict(loss=loss, inv_scaling=inv, probs=probs, loss_partial=part, dlogits=dlogits)


# --------------------------------------------------------------------------- classifier

def fc_amp_fwd(x, w, bias, y=None, relu=False, dropout_p=0.0, seed=0, offset=0, workspace=None, stream=None):
    """y = act(x W^T + bias) (FC_AMP_FWD + ReLU + dropout, fc_op.cpp:259-347).  x [batch, in], w [out, in] half
    (or both bfloat16), bias float."""
    if x.dtype not in DTYPE_CODE:
        raise TypeError(f"x: float16 or bfloat16 expected, got {x.dtype}")
    _need(x, x.dtype, "x", 2)
    _need(w, x.dtype, "w", 2)
    if bias is not None:
        _need(bias, torch.float32, "bias", 1)
    b, i_f = x.shape
    o_f = w.shape[0]
    if w.shape[1] != i_f:
        raise ValueError("fc_amp_fwd: w must be [out, in]")
    if y is None:
        y = torch.empty((b, o_f), dtype=x.dtype, device=x.device)
    lib = _lib.load()
    ws = (workspace or default_workspace()).ensure(lib.trb200_fc_amp_workspace_bytes(b, i_f, o_f))
    check(lib.trb200_fc_amp_fwd_dtype(_ptr(x), _ptr(w), _ptr(bias), _ptr(y), b, i_f, o_f, 1 if relu else 0,
                                      float(dropout_p), int(seed), int(offset), DTYPE_CODE[x.dtype], _ptr(ws), ws.numel(),
                                      _stream(stream)))
    return y


def fc_act_bwd(da, act, dz=None, scale=1.0, stream=None):
    """dz = act > 0 ? da * scale : 0 (ReLU + dropout backward from the layer's own output)."""
    _need(da, torch.float16, "da")
    _need(act, torch.float16, "act")
    dz = torch.empty_like(da) if dz is None else dz
    check(_lib.load().trb200_fc_act_bwd(_ptr(da), _ptr(act), _ptr(dz), da.numel(), float(scale), _stream(stream)))
    return dz


def fc_amp_bwd(dy, w, x, dx=None, dw=None, db=None, want_dx=True, act=None, act_scale=1.0, workspace=None, stream=None):
    """(dx, dw, db) of an FC layer (FC_AMP_BWD, fc_op.cpp:349-480): dw half [out, in], db float [out].  With act =
    x as the previous layer's forward wrote it (ReLU / dropout applied), dx also carries that activation's backward."""
    lib = _lib.load()
    if dy.dtype not in DTYPE_CODE:
        raise TypeError(f"dy: float16 or bfloat16 expected, got {dy.dtype}")
    _need(dy, dy.dtype, "dy", 2)
    _need(w, dy.dtype, "w", 2)
    _need(x, dy.dtype, "x", 2)
    b, o_f = dy.shape
    i_f = x.shape[1]
    if dw is None:
        dw = torch.empty((o_f, i_f), dtype=dy.dtype, device=dy.device)
    if dw.dtype not in (dy.dtype, torch.float32):
        raise TypeError("fc_amp_bwd: dw must be of the layer's 16-bit type or float")
    if db is None:
        db = torch.empty(o_f, dtype=torch.float32, device=dy.device)
    if dx is None and want_dx:
        dx = torch.empty((b, i_f), dtype=dy.dtype, device=dy.device)
    ws = (workspace or default_workspace()).ensure(lib.trb200_fc_amp_workspace_bytes(b, i_f, o_f))
    check(lib.trb200_fc_amp_bwd_dtype(_ptr(dy), _ptr(w), _ptr(x), _ptr(dx), _ptr(dw), 1 if dw.dtype == torch.float32 else 0,
                                      _ptr(db), _ptr(act), float(act_scale), b, i_f, o_f, DTYPE_CODE[dy.dtype],
                                      _ptr(ws), ws.numel(), _stream(stream)))
    return dx, dw, db


# --------------------------------------------------------------------------- all-reduce side

def scale_f32(t, factor, stream=None):
    _need(t, torch.float32, "t")
    check(_lib.load().trb200_scale_f32(_ptr(t), t.numel(), float(factor), _stream(stream)))
    return t


def cast_f16_to_f32(src, dst=None, factor=1.0, stream=None):
    _need(src, torch.float16, "src")
    if dst is None:
        dst = torch.empty(src.shape, dtype=torch.float32, device=src.device)
    check(_lib.load().trb200_cast_f16_to_f32(_ptr(src), _ptr(dst), src.numel(), float(factor), _stream(stream)))
    return dst


def mean_allreduce(flat_f32, group=None, stream=None):
    """RANGE_MEAN_ALLREDUCE (allreduce_op.cpp:37-105): in-place FP32 sum over the ranks
    with NCCL, then the 1/world scale kernel.  A single rank is a no-op, as in the
    reference when only one GPU is used."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return flat_f32
    dist.all_reduce(flat_f32, op=dist.ReduceOp.SUM, group=group)
    if flat_f32.is_cuda:
        scale_f32(flat_f32, 1.0 / dist.get_world_size(group), stream=stream)
    else:   # gloo ranks on CPU (tests): same arithmetic, no CUDA kernel involved
        flat_f32.mul_(1.0 / dist.get_world_size(group))
    return flat_f32
