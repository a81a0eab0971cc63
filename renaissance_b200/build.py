"""Builds renaissance_b200/lib/libtrb200.so from csrc/ with nvcc for sm_100a.

    python -m renaissance_b200.build [--force] [--verbose]

The library is built in-tree (it travels with the source tree; nothing is
installed into site-packages).  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
# development builds: TRB200_BUILD_TAG=name gives lib/libtrb200_name.so built with TRB200_EXTRA_NVCC_FLAGS
_TAG = os.environ.get("TRB200_BUILD_TAG", "")
LIB = os.path.join(LIB_DIR, f"libtrb200{'_' + _TAG if _TAG else ''}.so")
OBJ_DIR = os.path.join(HERE, "build" + ("_" + _TAG if _TAG else ""))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-I", os.path.join(ROOT, "include"), "-I", CSRC,
] + os.environ.get("TRB200_EXTRA_NVCC_FLAGS", "").split()


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = sorted(glob.glob(os.path.join(CSRC, "*.cuh"))) + [os.path.join(ROOT, "include", "trb200.h")]
    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    objs = []
    procs = []
    for src in sources:
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [_nvcc(), *NVCC_FLAGS, "-c", src, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
                print(" ".join(cmd))
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(out)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if force or procs or _stale(LIB, objs):
        cmd = [_nvcc(), "-Wno-deprecated-gpu-targets", "-shared", "-o", LIB, *objs, "-lcudart"]
        subprocess.check_call(cmd)
    if not _TAG:
        build_plugin(force or bool(procs))
    return LIB


PLUGIN_DIR = os.path.join(HERE, "plugin")
PLUGIN_LIB = os.path.join(LIB_DIR, "libtrb200_plugin.so")


def build_plugin(force: bool = False) -> str:
    """The operator-registry adapter and the test harness (host C++ only), linked against libtrb200.so."""
    srcs = [os.path.join(PLUGIN_DIR, f) for f in ("b200_ops.cpp", "harness.cpp")]
    deps = srcs + [os.path.join(PLUGIN_DIR, "tr_shim.h"), os.path.join(ROOT, "include", "trb200.h"), LIB]
    if force or _stale(PLUGIN_LIB, deps):
        cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O2", "-Xcompiler", "-fPIC",
               "-shared", "-o", PLUGIN_LIB, *srcs,
               "-I", os.path.join(ROOT, "include"), "-I", PLUGIN_DIR, "-L", LIB_DIR, "-ltrb200",
               "-Xlinker", "-rpath=$ORIGIN", "-lcudart"]
        # the all-reduce launcher calls NCCL (as the reference's does under TR_USE_NCCL) when the header is there
        if os.path.exists("/usr/include/nccl.h"):
            cmd += ["-DTR_USE_NCCL", "-lnccl"]
        subprocess.check_call(cmd)
    return PLUGIN_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
