"""CPU-only checks of the C-ABI library: it loads, exports every symbol that
include/trb200.h declares, and rejects bad arguments before touching a GPU."""
import ctypes as C
import os
import subprocess

import pytest

from renaissance_b200 import _lib


@pytest.fixture(scope="module")
def lib():
    from renaissance_b200 import build
    build.build()
    return _lib.load()


def test_every_declared_symbol_is_exported(lib):
    names = _lib.declared_symbols()
    assert len(names) >= 20
    out = subprocess.check_output(["nm", "-D", "--defined-only", _lib.LIB_PATH], text=True)
    exported = {line.split()[-1] for line in out.splitlines() if " T " in line}
    missing = [n for n in names if n not in exported]
    assert not missing, f"declared but not exported: {missing}"
    for n in names:
        assert hasattr(lib, n)


def test_version_and_error_text(lib):
    assert lib.trb200_version() >= 100
    assert isinstance(lib.trb200_last_error(), bytes)


def test_null_pointers_are_rejected_without_a_gpu(lib):
    rc = lib.trb200_bnrelu_bwd(None, None, None, None, None, None, None, None, None, 16, 64, None, 0, None)
    assert rc == _lib.ERR_INVALID_ARGUMENT
    assert b"null" in lib.trb200_last_error()
    rc = lib.trb200_softmax_ce_fwd(None, 8, None, None, None, 8, None, None, None, 4, 8, None)
    assert rc == _lib.ERR_INVALID_ARGUMENT
    rc = lib.trb200_cbr_bwd(None)
    assert rc == _lib.ERR_INVALID_ARGUMENT
    with pytest.raises(_lib.Trb200Error) as e:
        _lib.check(rc)
    assert e.value.code == _lib.ERR_INVALID_ARGUMENT


def test_bad_geometry_is_rejected(lib):
    d = _lib.ConvDesc(0, 8, 8, 64, 64, 3, 3, 1, 1, 1, 1)
    buf = C.c_void_p(256)
    assert lib.trb200_conv_wgrad(C.byref(d), buf, buf, buf, None, 0, None) == _lib.ERR_INVALID_ARGUMENT
    d = _lib.ConvDesc(1, 2, 2, 64, 64, 7, 7, 0, 0, 1, 1)      # filter larger than the input
    assert lib.trb200_conv_dgrad(C.byref(d), buf, buf, C.c_void_p(512), None, 0, None) == _lib.ERR_INVALID_ARGUMENT
    assert lib.trb200_bnrelu_bwd_workspace_bytes(100, 12) == 0     # c not a multiple of 8
    assert lib.trb200_set_conv_backend(7) == _lib.ERR_INVALID_ARGUMENT


def test_tensor_core_coverage_rule(lib):
    vgg = _lib.ConvDesc(256, 56, 56, 64, 64, 3, 3, 1, 1, 1, 1)
    first = _lib.ConvDesc(256, 224, 224, 4, 64, 3, 3, 1, 1, 1, 1)
    strided = _lib.ConvDesc(8, 56, 56, 64, 64, 3, 3, 1, 1, 2, 2)
    one_by_one = _lib.ConvDesc(8, 56, 56, 256, 64, 1, 1, 0, 0, 1, 1, 1)       # bfloat16
    stem = _lib.ConvDesc(8, 224, 224, 4, 64, 7, 7, 3, 3, 2, 2)
    stride_three = _lib.ConvDesc(8, 56, 56, 64, 64, 3, 3, 1, 1, 3, 3)
    odd = _lib.ConvDesc(8, 56, 56, 24, 64, 3, 3, 1, 1, 1, 1)
    for which in (0, 1, 2):
        assert lib.trb200_conv_uses_tensor_cores(C.byref(vgg), which) == 1
        # the 4-channel first layer: weight gradient and forward only (it has no data gradient)
        assert lib.trb200_conv_uses_tensor_cores(C.byref(first), which) == (0 if which == 1 else 1)
        # stride 2 runs on the same kernels through stepped tensor maps / parity classes; 1x1 is one tap
        assert lib.trb200_conv_uses_tensor_cores(C.byref(strided), which) == 1
        assert lib.trb200_conv_uses_tensor_cores(C.byref(one_by_one), which) == 1
        # a 7x7 first layer is lowered to rows and run as a 1x1 convolution (no data gradient)
        assert lib.trb200_conv_uses_tensor_cores(C.byref(stem), which) == (0 if which == 1 else 1)
        for direct in (stride_three, odd):
            assert lib.trb200_conv_uses_tensor_cores(C.byref(direct), which) == 0
    # the strided data gradient needs room for its filter view (nine taps in parity-class order)
    assert lib.trb200_conv_dgrad_workspace_bytes(C.byref(strided)) >= 9 * 64 * 64 * 2
    # channel counts the tiled kernels do not cover fall back to the stride-1 kernel plus a resampled tensor
    wide = _lib.ConvDesc(8, 56, 56, 64, 192, 3, 3, 1, 1, 2, 2)
    if lib.trb200_conv_uses_tensor_cores(C.byref(wide), 0):
        assert lib.trb200_conv_wgrad_workspace_bytes(C.byref(wide)) >= 8 * 56 * 56 * 192 * 2
    bad = _lib.ConvDesc(8, 56, 56, 64, 64, 3, 3, 1, 1, 1, 1, 7)
    assert lib.trb200_conv_wgrad_workspace_bytes(C.byref(bad)) == 0        # unknown dtype


def test_workspace_sizes_are_consistent(lib):
    d = _lib.ConvDesc(8, 28, 28, 128, 256, 3, 3, 1, 1, 1, 1)
    wg = lib.trb200_conv_wgrad_workspace_bytes(C.byref(d))
    dg = lib.trb200_conv_dgrad_workspace_bytes(C.byref(d))
    bn = lib.trb200_bnrelu_bwd_workspace_bytes(8 * 28 * 28, 256)
    total = lib.trb200_cbr_bwd_workspace_bytes(C.byref(d), 0)
    first = lib.trb200_cbr_bwd_workspace_bytes(C.byref(d), 1)
    assert wg > 0 and dg >= 9 * 128 * 256 * 2 and bn > 0
    assert total >= wg + dg + bn and first >= wg + bn and first < total


def test_registry_adapter_library_loads_and_exports_the_hook(lib):
    path = os.path.join(os.path.dirname(_lib.LIB_PATH), "libtrb200_plugin.so")
    assert os.path.exists(path)
    out = subprocess.check_output(["nm", "-D", "--defined-only", path], text=True)
    assert " T tr_b200_register_ops" in out
    plug = C.CDLL(path)
    assert hasattr(plug, "tr_b200_register_ops") and hasattr(plug, "trbh_create")


def test_product_package_never_imports_the_oracle():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    pkg = os.path.join(root, "renaissance_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), f"{f} mentions the oracle"


def test_adapter_compiles_against_the_reference_headers(tmp_path):
    """The registry adapter must keep compiling against the reference's own headers (the drop-in claim).  Needs a
    checkout of the reference: its path comes from TR_REFERENCE_ROOT; without one the test is skipped.  The
    reference's memory_arena.h includes mimalloc.h, which is not installed here: an empty header of that name stands
    in for it (the adapter uses none of it; this is a syntax check, nothing is linked)."""
    import shutil
    ref = os.environ.get("TR_REFERENCE_ROOT", "")
    if not ref or not os.path.isdir(os.path.join(ref, "include")):
        pytest.skip("TR_REFERENCE_ROOT does not name a checkout of the reference")
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("g++ not found")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = os.path.join(root, "renaissance_b200", "plugin", "b200_ops.cpp")
    (tmp_path / "mimalloc.h").write_text("")
    base = [gxx, "-std=c++17", "-fsyntax-only", "-DTRB200_WITH_REFERENCE_HEADERS", "-DTR_USE_CUDA",
            "-I", os.path.join(ref, "include"), "-I", os.path.join(root, "include"), "-I", "/usr/local/cuda/include",
            "-I", str(tmp_path), src]
    variants = [[]]
    if os.path.exists("/usr/include/nccl.h"):
        variants.append(["-DTR_USE_NCCL"])
    for extra in variants:
        res = subprocess.run(base + extra, capture_output=True, text=True)
        assert res.returncode == 0, res.stderr[-2000:]
