"""Builds libkleos_b200.so (CUDA kernels + C ABI) and the C++ driver kleos_driver in-tree with
nvcc for sm_100a."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libkleos_b200.so")
DRIVER = os.path.join(HERE, "kleos_driver")
SOURCES = ["kleos_api.cu"]


def _newest_source_mtime() -> float:
    newest = 0.0
    for root in (CSRC, os.path.join(os.path.dirname(HERE), "include")):
        for name in os.listdir(root):
            newest = max(newest, os.path.getmtime(os.path.join(root, name)))
    return newest


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_source_mtime():
        return LIB
    cmd = [
        "nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
        "-shared", "-Xcompiler", "-fPIC", "-ccbin", "g++",
        "-I", "/usr/include",  # nccl.h (types only; the library itself is dlopen'ed)
        "-o", LIB,
    ] + [os.path.join(CSRC, s) for s in SOURCES] + ["-ldl"]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    subprocess.check_call(cmd)
    return LIB


def build_driver(force: bool = False) -> str:
    """The stand-alone C++ driver on include/kleos_b200.hpp (host code only; links the library
    and finds it next to itself at run time)."""
    build()
    if not force and os.path.exists(DRIVER) and os.path.getmtime(DRIVER) >= _newest_source_mtime():
        return DRIVER
    subprocess.check_call([
        "nvcc", "-O2", "-std=c++17", "-Wno-deprecated-gpu-targets", "-ccbin", "g++",
        os.path.join(CSRC, "host_driver.cpp"),
        "-o", DRIVER, "-L", HERE, "-lkleos_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN",
    ])
    return DRIVER


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_driver(force="--force" in sys.argv))
