"""ctypes binding of libtrb200.so (the C ABI declared in include/trb200.h).

The library must exist: there is no fallback path.  ``load()`` raises if it is
missing; build it with ``python -m renaissance_b200.build``.
"""
from __future__ import annotations

import ctypes as C
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("TRB200_LIB") or os.path.join(_HERE, "lib", "libtrb200.so")
HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "trb200.h")

OK = 0
ERR_INVALID_ARGUMENT = -1
ERR_UNSUPPORTED = -2
ERR_WORKSPACE = -3
ERR_CUDA = -4
ERR_DEVICE_TIMEOUT = -5


class Trb200Error(RuntimeError):
    """A C-ABI call returned a non-zero status (the plugin's counterpart of the
    reference's TR_DEVICE_ERROR exception)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"trb200 error {code}: {message}")
        self.code = code


class ConvDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("n", "h", "w", "c", "k", "r", "s", "pad_h", "pad_w", "stride_h", "stride_w", "dtype")]


class CbrBwdArgs(C.Structure):
    _fields_ = [
        ("conv", ConvDesc),
        ("dy", C.c_void_p), ("w", C.c_void_p), ("gamma", C.c_void_p), ("saved_mean", C.c_void_p),
        ("saved_inv_std", C.c_void_p), ("mask_bits", C.c_void_p), ("x", C.c_void_p),
        ("dx", C.c_void_p), ("dw", C.c_void_p), ("dgamma", C.c_void_p), ("dbeta", C.c_void_p),
        ("conv_out", C.c_void_p), ("bn_scratch", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("stream_bn", C.c_void_p), ("stream_wgrad", C.c_void_p), ("stream_dgrad", C.c_void_p),
        ("ev_bn", C.c_void_p), ("ev_wgrad", C.c_void_p), ("ev_dgrad", C.c_void_p),
        ("pool_argmax", C.c_void_p),
        ("ev_time", C.c_void_p * 4),
    ]


_lib = None


def declared_symbols() -> list[str]:
    """Every function name that include/trb200.h declares."""
    text = open(HEADER_PATH).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(trb200_[a-z0-9_]+)\s*\(", text)))


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m renaissance_b200.build` "
            "(there is no CPU or PyTorch fallback for these operators)")
    lib = C.CDLL(LIB_PATH)
    vp, i32, i64, sz, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t, C.c_float
    pdesc = C.POINTER(ConvDesc)
    sig = {
        "trb200_last_error": (C.c_char_p, []),
        "trb200_version": (C.c_int, []),
        "trb200_device_arch": (C.c_int, []),
        "trb200_kernel_launch_count": (C.c_uint64, []),
        "trb200_device_status": (C.c_int, []),
        "trb200_selftest_wait_timeout": (C.c_int, [C.c_uint64, vp, vp]),
        "trb200_set_conv_backend": (C.c_int, [C.c_int]),
        "trb200_conv_uses_tensor_cores": (C.c_int, [pdesc, C.c_int]),
        "trb200_bnrelu_bwd_workspace_bytes": (sz, [i64, i32]),
        "trb200_bnrelu_bwd": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, vp, sz, vp]),
        "trb200_bnrelu_bwd_dtype": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, i32, vp, sz, vp]),
        "trb200_add16": (C.c_int, [vp, vp, vp, i64, i32, vp]),
        "trb200_add_relu_mask": (C.c_int, [vp, vp, vp, vp, i64, i32, vp]),
        "trb200_relu_mask_bwd": (C.c_int, [vp, vp, vp, i64, vp]),
        "trb200_maxpool_fwd": (C.c_int, [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, vp]),
        "trb200_maxpool_bwd": (C.c_int, [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, vp]),
        "trb200_avgpool_global_fwd": (C.c_int, [vp, vp, i32, i32, i32, i32, i32, vp]),
        "trb200_avgpool_global_bwd": (C.c_int, [vp, vp, i32, i32, i32, i32, i32, vp]),
        "trb200_bn_stats_finalize_dtype": (C.c_int, [vp, vp, vp, f32, f32, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32,
                                                    i32, vp, sz, vp]),
        "trb200_bn_apply_dtype": (C.c_int, [vp, vp, vp, vp, vp, i64, i32, i32, i32, vp]),
        "trb200_bnrelu_bwd_static": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, vp]),
        "trb200_conv_wgrad_workspace_bytes": (sz, [pdesc]),
        "trb200_conv_wgrad": (C.c_int, [pdesc, vp, vp, vp, vp, sz, vp]),
        "trb200_conv_dgrad_workspace_bytes": (sz, [pdesc]),
        "trb200_conv_dgrad": (C.c_int, [pdesc, vp, vp, vp, vp, sz, vp]),
        "trb200_conv_fprop_workspace_bytes": (sz, [pdesc]),
        "trb200_conv_fprop": (C.c_int, [pdesc, vp, vp, vp, vp, sz, vp]),
        "trb200_conv_fprop_bn_stats_workspace_bytes": (sz, [pdesc]),
        "trb200_conv_fprop_bn_stats": (C.c_int, [pdesc, vp, vp, vp, vp, vp, f32, f32, vp, vp, vp, vp, vp, vp, vp, vp,
                                                 vp, sz, vp]),
        "trb200_cbr_bwd_workspace_bytes": (sz, [pdesc, C.c_int]),
        "trb200_cbr_bwd": (C.c_int, [C.POINTER(CbrBwdArgs)]),
        "trb200_softmax_ce_fwd": (C.c_int, [vp, i64, vp, vp, vp, i64, vp, vp, vp, i32, i32, vp]),
        "trb200_softmax_ce_bwd": (C.c_int, [vp, i64, vp, vp, vp, vp, vp, i64, i32, i32, vp]),
        "trb200_softmax_ce_fused": (C.c_int, [vp, i64, vp, vp, vp, vp, i64, vp, i64, vp, vp, vp, i32, i32, vp]),
        "trb200_softmax_ce_fused_dtype": (C.c_int, [vp, i64, vp, vp, vp, vp, i64, vp, vp, vp, i32, i32, i32, vp]),
        "trb200_bn_stats_workspace_bytes": (sz, [i64, i32]),
        "trb200_bn_stats_finalize": (C.c_int, [vp, vp, vp, f32, f32, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32,
                                               vp, sz, vp]),
        "trb200_bn_apply_relu_mask": (C.c_int, [vp, vp, vp, vp, vp, i64, i32, vp]),
        "trb200_maxpool2x2_fwd": (C.c_int, [vp, vp, vp, i32, i32, i32, i32, vp]),
        "trb200_maxpool2x2_bwd": (C.c_int, [vp, vp, vp, i32, i32, i32, i32, vp]),
        "trb200_bn_apply_relu_mask_pool": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp]),
        "trb200_bnrelu_pool_bwd_workspace_bytes": (sz, [i32, i32, i32, i32]),
        "trb200_bnrelu_pool_bwd": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp, sz, vp]),
        "trb200_check_nonfinite": (C.c_int, [vp, i64, vp, vp]),
        "trb200_sgd_momentum": (C.c_int, [vp, vp, vp, vp, i64, f32, f32, f32, vp, vp, vp]),
        "trb200_sgd_nesterov": (C.c_int, [vp, vp, vp, vp, i64, f32, f32, f32, vp, vp, vp]),
        "trb200_sgd_plain": (C.c_int, [vp, vp, vp, i64, f32, f32, vp, vp, vp]),
        "trb200_check_nan_and_clip": (C.c_int, [vp, i64, f32, vp, vp]),
        "trb200_grad_scaling": (C.c_int, [vp, vp, i32, vp]),
        "trb200_fc_amp_workspace_bytes": (sz, [i32, i32, i32]),
        "trb200_fc_amp_fwd": (C.c_int, [vp, vp, vp, vp, i32, i32, i32, i32, f32, C.c_uint64, C.c_uint64, vp, sz, vp]),
        "trb200_fc_act_bwd": (C.c_int, [vp, vp, vp, i64, f32, vp]),
        "trb200_fc_amp_bwd": (C.c_int, [vp, vp, vp, vp, vp, i32, vp, vp, f32, i32, i32, i32, vp, sz, vp]),
        "trb200_fc_amp_fwd_dtype": (C.c_int, [vp, vp, vp, vp, i32, i32, i32, i32, f32, C.c_uint64, C.c_uint64, i32, vp, sz,
                                              vp]),
        "trb200_fc_amp_bwd_dtype": (C.c_int, [vp, vp, vp, vp, vp, i32, vp, vp, f32, i32, i32, i32, i32, vp, sz, vp]),
        "trb200_scale_f32": (C.c_int, [vp, i64, f32, vp]),
        "trb200_cast_f16_to_f32": (C.c_int, [vp, vp, i64, f32, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(code: int) -> None:
    if code != 0:
        raise Trb200Error(code, load().trb200_last_error().decode("utf-8", "replace"))
