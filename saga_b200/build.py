"""Builds libb200opt.so (the C-ABI library) in-tree with nvcc for sm_100a.

Run as ``python -m saga_b200.build``; ``__graft_entry__.build()`` calls
``build_library()``.  nvcc cross-compiles without a GPU.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libb200opt.so")

SOURCES = ["b200opt.cu", "host_logic.cpp", "nccl_path.cpp", "fabric.cpp", "checkpoint.cpp"]
HEADERS = ["fused_step.cuh", "staged_step.cuh", "nvls_step.cuh", "nccl_path.h", "fabric.h",
           os.path.join("..", "..", "include", "b200opt.h")]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; libb200opt.so cannot be built")


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force=False, verbose=False):
    """Compiles the library if any source is newer than it; returns its path."""
    if not force and not _stale():
        return LIB
    cmd = [
        _nvcc(), "-std=c++17", "-O3", "-lineinfo",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-Xcompiler", "-fPIC,-Wall,-fvisibility=hidden",
        "-Xptxas", "-v" if verbose else "-O3",
        "-shared", "-o", LIB,
    ] + [os.path.join(CSRC, s) for s in SOURCES] + ["-ldl"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building libb200opt.so")
    if verbose:
        sys.stderr.write(res.stdout + res.stderr)
    return LIB


DRIVER = os.path.join(HERE, "host", "mt_driver")


def build_driver(force=False):
    """Compiles host/mt_driver (Saga's one-thread-per-GPU model over the C ABI)."""
    src = os.path.join(HERE, "host", "mt_driver.cpp")
    hdr = os.path.join(HERE, "host", "b200_adam_op.hpp")
    build_library()
    if not force and os.path.exists(DRIVER) and all(
            os.path.getmtime(DRIVER) > os.path.getmtime(f) for f in (src, hdr, LIB)):
        return DRIVER
    cmd = [_nvcc(), "-std=c++17", "-O2", "-x", "cu", src, "-o", DRIVER,
           "-I", os.path.join(HERE, "..", "include"), "-I", os.path.join(HERE, "host"),
           "-L", HERE, "-lb200opt", "-Xlinker", "-rpath," + "$ORIGIN/..", "-lpthread"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building mt_driver")
    return DRIVER


if __name__ == "__main__":
    print(build_library(force=True, verbose="-v" in sys.argv))
    print(build_driver(force=True))
