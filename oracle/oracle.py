"""numpy front end of the CPU oracle (``oracle/trb_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()``
and by ``bench.py``'s CPU-baseline legs, never by the product package.

Arrays are NHWC / KRSC and compact.  Half tensors are ``np.float16`` arrays.
Each wrapper names the reference lines its C function restates; see the header
of ``trb_oracle.c`` for the full list.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libtrb_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside this file."""
    src = os.path.join(_HERE, "trb_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-s"] + (["-B"] if force else []))
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _f16(a):
    return np.ascontiguousarray(a, dtype=np.float16)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(C.c_int(n))


def out_hw(h, w, r, s, pad, stride):
    pad, stride = int(pad), int(stride)
    return (h + 2 * pad - r) // stride + 1, (w + 2 * pad - s) // stride + 1


# --------------------------------------------------------------------------- masks

def mask_pack(mask_bytes: np.ndarray) -> np.ndarray:
    """0/1 byte mask -> cuDNN BOOLEAN bits, LSB first (cbr_amp_test_utils.hpp:131-145)."""
    m = np.ascontiguousarray(mask_bytes, dtype=np.int8).ravel()
    bits = np.zeros((m.size + 7) // 8, dtype=np.uint8)
    lib().orc_mask_pack(_p(m), _p(bits), C.c_int64(m.size))
    return bits


def mask_unpack(bits: np.ndarray, n: int) -> np.ndarray:
    """cuDNN BOOLEAN bits -> 0/1 bytes (cbr_amp_test_utils.hpp:115-127)."""
    b = np.ascontiguousarray(bits, dtype=np.uint8).ravel()
    out = np.zeros(n, dtype=np.int8)
    lib().orc_mask_unpack(_p(b), _p(out), C.c_int64(n))
    return out


# --------------------------------------------------------------------------- conv fp32

def conv_fwd(x, w, pad=1, stride=1):
    """conv_op.cpp:664-729."""
    x, w = _f32(x), _f32(w)
    n, h, ww, c = x.shape
    k, r, s, _ = w.shape
    oh, ow = out_hw(h, ww, r, s, pad, stride)
    y = np.empty((n, oh, ow, k), np.float32)
    lib().orc_conv_fwd_f32(_p(x), _p(w), _p(y), n, h, ww, c, k, r, s, int(pad), int(stride))
    return y


def conv_dgrad(dy, w, x_shape, pad=1, stride=1):
    """conv_op.cpp:776-812."""
    dy, w = _f32(dy), _f32(w)
    n, h, ww, c = x_shape
    k, r, s, _ = w.shape
    dx = np.empty(x_shape, np.float32)
    lib().orc_conv_dgrad_f32(_p(dy), _p(w), _p(dx), n, h, ww, c, k, r, s, int(pad), int(stride))
    return dx


def conv_wgrad(dy, x, w_shape, pad=1, stride=1):
    """conv_op.cpp:814-848."""
    dy, x = _f32(dy), _f32(x)
    n, h, ww, c = x.shape
    k, r, s, _ = w_shape
    dw = np.empty(w_shape, np.float32)
    lib().orc_conv_wgrad_f32(_p(dy), _p(x), _p(dw), n, h, ww, c, k, r, s, int(pad), int(stride))
    return dw


# --------------------------------------------------------------------------- BN / ReLU fp32

def bn_fwd(x, gamma, beta, running_mean=None, running_var=None, eps=1e-5, momentum=0.1):
    """bn_op.cpp:55-116.  Returns (y, saved_mean, saved_inv_std); running stats updated in place."""
    x = _f32(x)
    cch = x.shape[-1]
    m = x.size // cch
    y = np.empty_like(x)
    mean = np.empty(cch, np.float32)
    inv = np.empty(cch, np.float32)
    lib().orc_bn_fwd_f32(_p(x), _p(_f32(gamma)), _p(_f32(beta)), _p(running_mean), _p(running_var),
                         _p(y), _p(mean), _p(inv), C.c_int64(m), cch, C.c_float(eps), C.c_float(momentum))
    return y, mean, inv


def bn_bwd(dy, x, gamma, saved_mean, saved_inv_std):
    """bn_op.cpp:119-168.  Returns (dx, dgamma, dbeta)."""
    dy, x = _f32(dy), _f32(x)
    cch = x.shape[-1]
    m = x.size // cch
    dx = np.empty_like(x)
    dg = np.empty(cch, np.float32)
    db = np.empty(cch, np.float32)
    lib().orc_bn_bwd_f32(_p(dy), _p(x), _p(_f32(gamma)), _p(_f32(saved_mean)), _p(_f32(saved_inv_std)),
                         _p(dx), _p(dg), _p(db), C.c_int64(m), cch)
    return dx, dg, db


def relu_fwd(x):
    """relu_op.cpp:348-371.  Returns (y, byte mask)."""
    x = _f32(x)
    y = np.empty_like(x)
    mask = np.empty(x.shape, np.int8)
    lib().orc_relu_fwd_f32(_p(x), _p(y), _p(mask), C.c_int64(x.size))
    return y, mask


def relu_bwd(dy, mask):
    """relu_op.cpp:398-419."""
    dy = _f32(dy)
    mask = np.ascontiguousarray(mask, dtype=np.int8)
    dx = np.empty_like(dy)
    lib().orc_relu_bwd_f32(_p(dy), _p(mask), _p(dx), C.c_int64(dy.size))
    return dx


# --------------------------------------------------------------------------- softmax-CE

def softmax_ce_fwd_cpu(logits, labels, scaling=1.0, ls=0.0, loss_init=0.0):
    """CPU operator, softmax_ce_op.cpp:114-156.  Returns (loss, inv_scaling, probs)."""
    z = _f32(logits)
    b, k = z.shape
    loss = np.array([loss_init], np.float32)
    inv = np.zeros(1, np.float32)
    probs = np.empty_like(z)
    lib().orc_softmax_ce_fwd_cpu(_p(z), _p(_i32(labels)), _p(loss), _p(inv), _p(probs),
                                 b, k, C.c_float(scaling), C.c_float(ls))
    return float(loss[0]), float(inv[0]), probs


def softmax_ce_bwd(probs, labels, scale, ls=0.0):
    """softmax_ce_op.cpp:237-256 / softmax_ce_op.cu:438-468 (fp32 output)."""
    p = _f32(probs)
    b, k = p.shape
    d = np.empty_like(p)
    lib().orc_softmax_ce_bwd(_p(p), _p(_i32(labels)), _p(d), b, k, C.c_float(scale), C.c_float(ls))
    return d


def softmax_ce_amp(logits16, labels, scaling=1.0, ls=0.0, want_probs=True, want_grad=True):
    """GPU AMP operator semantics, softmax_ce_op.cu:63-177, 372-468.

    Returns dict(probs fp32, loss_partial fp32[B], loss, inv_scaling, dlogits fp16)."""
    z = _f16(logits16)
    b, k = z.shape
    probs = np.empty((b, k), np.float32) if want_probs else None
    part = np.empty(b, np.float32)
    loss = np.zeros(1, np.float32)
    inv = np.zeros(1, np.float32)
    d = np.empty((b, k), np.float16) if want_grad else None
    lib().orc_softmax_ce_amp(_p(z), C.c_int64(k), _p(_i32(labels)), _p(probs), _p(part), _p(loss), _p(inv),
                             _p(d), C.c_int64(k), b, k, C.c_float(scaling), C.c_float(ls))
    return dict(probs=probs, loss_partial=part, loss=float(loss[0]), inv_scaling=float(inv[0]), dlogits=d)


# --------------------------------------------------------------------------- FC / SGD

def fc_fwd(x, w, b=None):
    """fc_op.cpp:802-832."""
    x, w = _f32(x), _f32(w)
    y = np.empty((x.shape[0], w.shape[0]), np.float32)
    lib().orc_fc_fwd_f32(_p(x), _p(w), _p(None if b is None else _f32(b)), _p(y),
                         x.shape[0], x.shape[1], w.shape[0])
    return y


def fc_bwd(dy, w, x, bias=True):
    """fc_op.cpp:835-898.  Returns (dx, dw, db)."""
    dy, w, x = _f32(dy), _f32(w), _f32(x)
    dx = np.empty_like(x)
    dw = np.empty_like(w)
    db = np.empty(w.shape[0], np.float32) if bias else None
    lib().orc_fc_bwd_f32(_p(dy), _p(w), _p(x), _p(dx), _p(dw), _p(db), x.shape[0], x.shape[1], w.shape[0])
    return dx, dw, db


def sgd(w, g, lr, wd=0.0, scaling=1.0):
    """optimizer_op.cpp:297-304 (in place on a float32 copy, returned)."""
    w = _f32(w).copy()
    lib().orc_sgd_f32(_p(w), _p(_f32(g)), C.c_int64(w.size), C.c_float(lr), C.c_float(wd), C.c_float(scaling))
    return w


def momentum(w, g, m, lr, wd=0.0, beta=0.9, scaling=1.0):
    """optimizer_op.cpp:306-313.  Returns (w, m)."""
    w, m = _f32(w).copy(), _f32(m).copy()
    lib().orc_momentum_f32(_p(w), _p(_f32(g)), _p(m), C.c_int64(w.size), C.c_float(lr), C.c_float(wd),
                           C.c_float(beta), C.c_float(scaling))
    return w, m


def nesterov(w, g, m, lr, wd=0.0, beta=0.9, scaling=1.0):
    """optimizer_op.cu:68-93.  Returns (w, m)."""
    w, m = _f32(w).copy(), _f32(m).copy()
    lib().orc_nesterov_f32(_p(w), _p(_f32(g)), _p(m), C.c_int64(w.size), C.c_float(lr), C.c_float(wd),
                           C.c_float(beta), C.c_float(scaling))
    return w, m


def check_nan_and_clip(g, clip):
    """check_op.cu:54-79.  Returns (clipped copy, flag)."""
    g = _f32(g).copy()
    fn = lib().orc_check_nan_and_clip_f32
    fn.restype = C.c_int
    return g, int(fn(_p(g), C.c_int64(g.size), C.c_float(clip)))


def grad_scaling(has_nan, scaling):
    """grad_scaling_op.cu:15-22."""
    fn = lib().orc_grad_scaling
    fn.restype = C.c_float
    return float(fn(C.c_int(int(has_nan)), C.c_float(scaling)))


# --------------------------------------------------------------------------- fused AMP block

def cbr_fwd_amp(x16, w16, gamma, beta, pad=1, stride=1, eps=1e-5, momentum=0.1,
                running_mean=None, running_var=None, round_steps=True, stats_from_half=False):
    """cbr_op.cpp:430-718.  Returns dict of conv_out, sum, sqsum, saved_mean, saved_inv_std,
    eq_scale, eq_bias, relu_out, mask_bits."""
    x, w = _f16(x16), _f16(w16)
    n, h, ww, c = x.shape
    k, r, s, _ = w.shape
    oh, ow = out_hw(h, ww, r, s, pad, stride)
    ne = n * oh * ow * k
    out = dict(
        conv_out=np.empty((n, oh, ow, k), np.float16),
        sum=np.empty(k, np.float32), sqsum=np.empty(k, np.float32),
        saved_mean=np.empty(k, np.float32), saved_inv_std=np.empty(k, np.float32),
        eq_scale=np.empty(k, np.float32), eq_bias=np.empty(k, np.float32),
        relu_out=np.empty((n, oh, ow, k), np.float16),
        mask_bits=np.zeros((ne + 7) // 8, np.uint8),
    )
    lib().orc_cbr_fwd_amp(_p(x), _p(w), _p(_f32(gamma)), _p(_f32(beta)), _p(running_mean), _p(running_var),
                          _p(out["conv_out"]), _p(out["sum"]), _p(out["sqsum"]),
                          _p(out["saved_mean"]), _p(out["saved_inv_std"]),
                          _p(out["eq_scale"]), _p(out["eq_bias"]), _p(out["relu_out"]), _p(out["mask_bits"]),
                          n, h, ww, c, k, r, s, int(pad), int(stride), C.c_float(eps), C.c_float(momentum),
                          1 if round_steps else 0, 1 if stats_from_half else 0)
    return out


def bnrelu_bwd_amp(dy16, mask_bits, conv_out16, gamma, saved_mean, saved_inv_std, want_dx=True):
    """cbr_op.cpp:1259-1353.  Returns (dconv fp16 or None, dgamma, dbeta)."""
    dy, x = _f16(dy16), _f16(conv_out16)
    cch = dy.shape[-1]
    m = dy.size // cch
    dconv = np.empty(dy.shape, np.float16) if want_dx else None
    dg = np.empty(cch, np.float32)
    db = np.empty(cch, np.float32)
    bits = np.ascontiguousarray(mask_bits, dtype=np.uint8)
    lib().orc_bnrelu_bwd_amp(_p(dy), _p(bits), _p(x), _p(_f32(gamma)), _p(_f32(saved_mean)),
                             _p(_f32(saved_inv_std)), _p(dconv), _p(dg), _p(db), C.c_int64(m), cch)
    return dconv, dg, db


def cbr_bwd_amp(dy16, w16, gamma, saved_mean, saved_inv_std, mask_bits, x16, conv_out16,
                pad=1, stride=1, first_layer=False):
    """cbr_op.cpp:1359-1651.  Returns dict(dx, dw, dgamma, dbeta, dconv)."""
    dy, w, x, co = _f16(dy16), _f16(w16), _f16(x16), _f16(conv_out16)
    n, h, ww, c = x.shape
    k, r, s, _ = w.shape
    dx = None if first_layer else np.empty(x.shape, np.float16)
    dw = np.empty(w.shape, np.float16)
    dg = np.empty(k, np.float32)
    db = np.empty(k, np.float32)
    dconv = np.empty(dy.shape, np.float16)
    bits = np.ascontiguousarray(mask_bits, dtype=np.uint8)
    lib().orc_cbr_bwd_amp(_p(dy), _p(w), _p(_f32(gamma)), _p(_f32(saved_mean)), _p(_f32(saved_inv_std)),
                          _p(bits), _p(x), _p(co), _p(dx), _p(dw), _p(dg), _p(db), _p(dconv),
                          n, h, ww, c, k, r, s, int(pad), int(stride))
    return dict(dx=dx, dw=dw, dgamma=dg, dbeta=db, dconv=dconv)


# --------------------------------------------------------------------------- max pooling

def maxpool2x2_fwd(x16):
    """maxpool_op.cu:23-150 (2x2, stride 2).  Returns (y fp16, argmax uint8 = kh*2+kw)."""
    x = _f16(x16)
    n, h, w, c = x.shape
    y = np.empty((n, h // 2, w // 2, c), np.float16)
    am = np.empty(y.shape, np.uint8)
    lib().orc_maxpool2x2_fwd_h16(_p(x), _p(y), _p(am), n, h, w, c)
    return y, am


def maxpool2x2_bwd(dy16, argmax, x_shape):
    """maxpool_op.cu:155-217."""
    dy = _f16(dy16)
    am = np.ascontiguousarray(argmax, dtype=np.uint8)
    dx = np.empty(x_shape, np.float16)
    n, h, w, c = x_shape
    lib().orc_maxpool2x2_bwd_h16(_p(dy), _p(am), _p(dx), n, h, w, c)
    return dx


# --------------------------------------------------------------------------- general pooling (numpy restatements)

def maxpool_fwd(x, k, stride, pad):
    """maxpool_amp_fwd_mask_kernel, maxpool_op.cu:83-133: first maximum wins (strict >, in float), mask byte
    kh*k + kw, -1 (0xff) for a window with no pixel inside the image.  x: [n,h,w,c] float.  Returns (y, argmax uint8)."""
    x = np.asarray(x, np.float32)
    n, h, w, c = x.shape
    oh, ow = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
    best = np.full((n, oh, ow, c), -np.inf, np.float32)
    pos = np.full((n, oh, ow, c), -1, np.int32)
    for kh in range(k):
        for kw in range(k):
            for o_h in range(oh):
                ih = o_h * stride - pad + kh
                if ih < 0 or ih >= h:
                    continue
                for o_w in range(ow):
                    iw = o_w * stride - pad + kw
                    if iw < 0 or iw >= w:
                        continue
                    v = x[:, ih, iw, :]
                    gt = v > best[:, o_h, o_w, :]
                    best[:, o_h, o_w, :] = np.where(gt, v, best[:, o_h, o_w, :])
                    pos[:, o_h, o_w, :] = np.where(gt, kh * k + kw, pos[:, o_h, o_w, :])
    return best, (pos & 0xff).astype(np.uint8)


def maxpool_bwd(dy, argmax, x_shape, k, stride, pad):
    """maxpool_bwd_deterministic_kernel, maxpool_op.cu:155-217: float gather per input pixel in (oh, ow) order."""
    dy = np.asarray(dy, np.float32)
    n, h, w, c = x_shape
    _, oh, ow, _ = dy.shape
    dx = np.zeros(x_shape, np.float32)
    for o_h in range(oh):
        for o_w in range(ow):
            a = argmax[:, o_h, o_w, :].astype(np.int32)
            for kh in range(k):
                ih = o_h * stride - pad + kh
                if ih < 0 or ih >= h:
                    continue
                for kw in range(k):
                    iw = o_w * stride - pad + kw
                    if iw < 0 or iw >= w:
                        continue
                    dx[:, ih, iw, :] += np.where(a == kh * k + kw, dy[:, o_h, o_w, :], np.float32(0))
    return dx


def avgpool_global_fwd(x):
    """gap_op.cpp:137-155: y = (sum over h, w) * (1 / (h*w)), float."""
    x = np.asarray(x, np.float32)
    n, h, w, c = x.shape
    acc = np.zeros((n, c), np.float32)
    for i in range(h):
        for j in range(w):
            acc += x[:, i, j, :]
    return acc * np.float32(1.0 / (h * w))


def avgpool_global_bwd(dy, h, w):
    """gap_op.cu:92-112: dx = dy * (1 / (h*w)) at every pixel."""
    dy = np.asarray(dy, np.float32)
    return np.broadcast_to((dy * np.float32(1.0 / (h * w)))[:, None, None, :], (dy.shape[0], h, w, dy.shape[1])).copy()
