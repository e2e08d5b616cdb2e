"""In-tree build of the native libraries (no cmake, no JIT cache).

    python -m ms_custom_ops_b200.build [--force]

libmsco_b200.so          CUDA kernels + thin C ABI      nvcc, sm_100a only
libms_custom_ops_host.so C++ operator layer             g++, links the kernel library

bench/msco_bench         standalone C++ benchmark       nvcc, links the kernel library

All land inside this package so that they travel with the source tree.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
INCLUDE = os.path.join(ROOT, "include")
CSRC = os.path.join(HERE, "csrc")
OPS = os.path.join(HERE, "ops")

KERNEL_LIB = os.path.join(HERE, "libmsco_b200.so")
HOST_LIB = os.path.join(HERE, "libms_custom_ops_host.so")

NVCC_FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "-shared", "--threads", "4"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd):
    print("+", " ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)


def build_kernels(force=False, verbose_ptxas=False):
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    deps = srcs + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + \
        glob.glob(os.path.join(INCLUDE, "*.h"))
    if not force and not _stale(KERNEL_LIB, deps):
        return KERNEL_LIB
    cmd = [_nvcc()] + NVCC_FLAGS + ["-I", INCLUDE, "-I", CSRC]
    if verbose_ptxas:
        cmd += ["-Xptxas", "-v"]
    _run(cmd + ["-o", KERNEL_LIB] + srcs)
    return KERNEL_LIB


def build_host(force=False):
    srcs = sorted(glob.glob(os.path.join(OPS, "**", "*.cc"), recursive=True))
    if not srcs:
        return None
    deps = srcs + glob.glob(os.path.join(OPS, "**", "*.h"), recursive=True) + glob.glob(os.path.join(INCLUDE, "*.h"))
    if not force and not _stale(HOST_LIB, deps + [KERNEL_LIB]):
        return HOST_LIB
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-Wall", "-I", INCLUDE, "-I", HERE,
           "-o", HOST_LIB] + srcs + ["-L", HERE, "-lmsco_b200", "-Wl,-rpath,$ORIGIN", "-lpthread"]
    _run(cmd)
    return HOST_LIB


def build_bench(force=False):
    """Standalone C++ benchmark harness (no Python at run time): bench/msco_bench."""
    src = os.path.join(HERE, "bench", "msco_bench.cu")
    exe = os.path.join(HERE, "bench", "msco_bench")
    if not os.path.exists(src):
        return None
    if not force and not _stale(exe, [src, KERNEL_LIB, os.path.join(INCLUDE, "msco_b200.h")]):
        return exe
    _run([_nvcc(), "-std=c++17", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", "-I", INCLUDE, "-o", exe, src,
          "-L", HERE, "-lmsco_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/.."])
    return exe


def build_all(force=False, verbose_ptxas=False):
    build_kernels(force, verbose_ptxas)
    build_host(force)
    build_bench(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose_ptxas="--ptxas-v" in sys.argv)
