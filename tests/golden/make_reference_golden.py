#!/usr/bin/env python3
"""Golden vectors made by the REFERENCE project's own generator scripts.

The reference's operator tests take their expected values from Python scripts
that sit beside the C++ drivers; each script writes its tensors as ``.tsr``
files which the C++ test then reads.  This script imports those generators
unchanged from a checkout of the reference, runs them on small shapes, reads
the ``.tsr`` files back with the reference's own reader and stores every
tensor of a case in one ``ref_<case>.npz``:

    generator (path inside the reference)       function            cases
    tests/op/test_conv_fwd_bwd.py               generate            ref_conv_*
    tests/op/test_bn_fwd_bwd_legacy.py          generate            ref_bn_*
    tests/correction/test_softmax_ce.py         generate_reference_data   ref_softmax_*
    tests/op/test_maxpool_fwd_bwd.py            generate            ref_maxpool_*
    tests/correction/test_mlp_final.py          generate            ref_mlp_final_fp32
    python/scripts/tsr_v4.py                    load_single_tensor  (reader)

    TR_REFERENCE_ROOT=/path/to/renaissance python tests/golden/make_reference_golden.py

Nothing of the reference is copied: the scripts run where they lie.  The
fixtures travel with this repository, the reference checkout does not, so the
tests only ever read the ``.npz`` files.  Nothing here imports the oracle or
the CUDA library.
"""
import glob
import importlib.util
import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
torch.set_num_threads(1)


def reference_root():
    root = os.environ.get("TR_REFERENCE_ROOT")
    if not root or not os.path.isdir(root):
        sys.exit("set TR_REFERENCE_ROOT to a checkout of tech-renaissance/renaissance")
    return root


def load_module(root, rel):
    path = os.path.join(root, rel)
    name = "trref_" + os.path.splitext(os.path.basename(rel))[0]
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def collect(ws, reader):
    """Every .tsr of a generator's workspace, keyed by file name without the
    extension; shapes are the reference's 4-D NHWC shapes."""
    out = {}
    for path in sorted(glob.glob(os.path.join(ws, "*.tsr"))):
        out[os.path.splitext(os.path.basename(path))[0]] = np.ascontiguousarray(reader(path))
    return out


def save(name, script, call, arrays, **extra):
    arrays = dict(arrays)
    arrays.update(extra)
    arrays["provenance"] = np.array(f"{script}::{call}")
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **arrays)
    print(f"{name}.npz  {os.path.getsize(path) / 1024:.1f} KiB  <- {script}::{call}")


def main():
    root = reference_root()
    sys.path.insert(0, os.path.join(root, "python", "scripts"))
    tsr = load_module(root, "python/scripts/tsr_v4.py")
    reader = tsr.load_single_tensor

    conv = load_module(root, "tests/op/test_conv_fwd_bwd.py")
    # (name, batch, IH, IW, C, K, kernel, stride, pad, seed, dtype)
    conv_cases = [
        ("ref_conv_fp32_3x3_s1", 2, 8, 8, 8, 16, 3, 1, 1, 42, "fp32"),
        ("ref_conv_fp32_3x3_s2", 2, 9, 7, 4, 8, 3, 2, 1, 43, "fp32"),
        ("ref_conv_fp32_1x1_s1", 2, 6, 6, 16, 8, 1, 1, 0, 44, "fp32"),
        ("ref_conv_fp32_7x7_s2", 1, 11, 11, 4, 8, 7, 2, 3, 45, "fp32"),
        ("ref_conv_fp16_3x3_s1", 2, 8, 8, 16, 16, 3, 1, 1, 46, "fp16"),
        # the smallest shape the tensor-core kernels take (64 channels in and out)
        ("ref_conv_fp16_3x3_s1_c64", 1, 8, 8, 64, 64, 3, 1, 1, 47, "fp16"),
    ]
    for name, b, ih, iw, c, k, ker, st, pad, seed, dt in conv_cases:
        with tempfile.TemporaryDirectory() as ws:
            conv.generate(b, ih, iw, c, k, ker, st, pad, seed, ws, dt)
            save(name, "tests/op/test_conv_fwd_bwd.py", f"generate({b},{ih},{iw},{c},{k},{ker},{st},{pad},{seed},ws,'{dt}')",
                 collect(ws, reader),
                 params=np.array([b, ih, iw, c, k, ker, st, pad, int(dt == "fp16")], np.int32))

    bn = load_module(root, "tests/op/test_bn_fwd_bwd_legacy.py")
    for name, is1d, b, h, w, c, seed, dt in [("ref_bn2d_fp32", False, 4, 5, 5, 8, 42, "fp32"),
                                             ("ref_bn1d_fp32", True, 16, 1, 1, 10, 43, "fp32"),
                                             ("ref_bn2d_fp16", False, 4, 6, 6, 16, 44, "fp16")]:
        with tempfile.TemporaryDirectory() as ws:
            bn.generate(is1d, b, h, w, c, 1e-5, 0.1, seed, ws, dt)
            save(name, "tests/op/test_bn_fwd_bwd_legacy.py", f"generate({is1d},{b},{h},{w},{c},1e-5,0.1,{seed},ws,'{dt}')",
                 collect(ws, reader), params=np.array([b, 1 if is1d else h, 1 if is1d else w, c], np.int32))

    sm = load_module(root, "tests/correction/test_softmax_ce.py")
    for name, b, classes, seed, dt in [("ref_softmax_fp32_1000", 8, 1000, 42, "fp32"),
                                       ("ref_softmax_fp16_1000", 8, 1000, 43, "fp16"),
                                       ("ref_softmax_fp32_10", 16, 10, 44, "fp32")]:
        with tempfile.TemporaryDirectory() as ws:
            sm.generate_reference_data(b, classes, seed, ws, dt)
            save(name, "tests/correction/test_softmax_ce.py", f"generate_reference_data({b},{classes},{seed},ws,'{dt}')",
                 collect(ws, reader), params=np.array([b, classes, int(dt == "fp16")], np.int32))

    mp = load_module(root, "tests/op/test_maxpool_fwd_bwd.py")
    for name, shape, k, st, pad, seed, dt in [("ref_maxpool_fp16_2x2_s2", (2, 8, 8, 8), 2, 2, 0, 42, "fp16"),
                                              ("ref_maxpool_fp16_3x3_s2", (2, 9, 9, 8), 3, 2, 1, 43, "fp16"),
                                              ("ref_maxpool_fp32_2x2_s2", (2, 6, 6, 8), 2, 2, 0, 44, "fp32")]:
        with tempfile.TemporaryDirectory() as ws:
            mp.generate(shape, k, st, pad, seed, ws, dt)
            save(name, "tests/op/test_maxpool_fwd_bwd.py", f"generate({shape},{k},{st},{pad},{seed},ws,'{dt}')",
                 collect(ws, reader), params=np.array([*shape, k, st, pad, int(dt == "fp16")], np.int32))

    mlp = load_module(root, "tests/correction/test_mlp_final.py")
    with tempfile.TemporaryDirectory() as ws:
        mlp.generate(42, ws, "fp32")
        arrays = collect(ws, reader)
        # the 784x512 first layer and the second layer's weight gradient are kept as their first
        # 32 output rows (the tests slice d_fc1 / d_fc2 the same way); every other tensor is whole
        arrays["w1_fp32"] = arrays["w1_fp32"][:32].copy()
        arrays["dw1_ref_fp32"] = arrays["dw1_ref_fp32"][:32].copy()
        arrays["dw2_ref_fp32"] = arrays["dw2_ref_fp32"][:32].copy()
        save("ref_mlp_final_fp32", "tests/correction/test_mlp_final.py", "generate(42,ws,'fp32')", arrays)


if __name__ == "__main__":
    main()
