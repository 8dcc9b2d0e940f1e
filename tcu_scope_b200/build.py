"""Builds libtcu_scope.so (the C-ABI CUDA library) for sm_100a, in-tree, with nvcc.

Run as ``python tcu_scope_b200/build.py`` (a plain script: it must work while
the library is missing or stale, when the package itself refuses to import).
nvcc cross-compiles, so this works on a machine without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libtcu_scope.so")
BENCH_PATH = os.path.join(PKG_DIR, "tcu_bench")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return nvcc


def _newer_than(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _sources() -> list[str]:
    out = [os.path.join(PKG_DIR, "..", "include", "tcu_scope.h")]
    for name in sorted(os.listdir(CSRC)):
        out.append(os.path.join(CSRC, name))
    return out


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile csrc/capi.cu (which includes every kernel; fp16 inputs) and csrc/capi_bf16.cu (the
    same sources for bf16 inputs) into libtcu_scope.so."""
    srcs = _sources()
    if not force and _newer_than(LIB_PATH, srcs):
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS, "--threads", "2", "-shared", "-o", LIB_PATH,
           os.path.join(CSRC, "capi.cu"), os.path.join(CSRC, "capi_bf16.cu")]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    subprocess.run(cmd, check=True)
    return LIB_PATH


def build_bench(force: bool = False) -> str:
    """Compile the C++ benchmark runner that registers the reference's benchmark names."""
    src = os.path.join(CSRC, "bench_main.cpp")
    if not os.path.exists(src):
        return ""
    if not force and _newer_than(BENCH_PATH, _sources()):
        return BENCH_PATH
    build_library(force=False)
    cmd = [_nvcc(), "-O2", "-std=c++17", "-o", BENCH_PATH, src,
           "-L" + PKG_DIR, "-ltcu_scope", "-Xlinker", "-rpath=$ORIGIN"]
    subprocess.run(cmd, check=True)
    return BENCH_PATH


if __name__ == "__main__":
    build_library(force="--force" in sys.argv, verbose="-v" in sys.argv)
    build_bench(force="--force" in sys.argv)
    print(LIB_PATH)
