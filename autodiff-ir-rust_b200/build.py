"""Builds libadb200.so in-tree (csrc/ -> autodiff-ir-rust_b200/libadb200.so) with nvcc for sm_100a.

    python autodiff-ir-rust_b200/build.py [--force] [--verbose]

nvcc cross-compiles without a GPU; the result travels with the source tree.  NVRTC is linked
dynamically from the CUDA toolkit (the generated kernels are compiled at first use), cudart is linked
statically, libcuda and libnccl are not linked at all (entry points are fetched at run time).
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libadb200.so")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")
SOURCES = ["adb_runtime.cu", "adb_gemm.cu", "adb_noalloc.cu", "adb_lower.cpp", "adb_codegen.cpp", "adb_shard.cpp"]


def needs_build() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    for root in (CSRC, os.path.join(os.path.dirname(HERE), "include")):
        for f in os.listdir(root):
            if os.path.getmtime(os.path.join(root, f)) > t:
                return True
    return False


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return OUT
    cmd = [
        os.path.join(CUDA, "bin", "nvcc"), "-O3", "-std=c++17",
        "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
        "-Xcompiler", "-fPIC,-Wall,-Wextra,-Wno-unused-parameter", "-shared",
        "-o", OUT,
    ] + [os.path.join(CSRC, s) for s in SOURCES] + [
        "-lnvrtc", "-ldl", "-Xlinker", f"-rpath={CUDA}/lib64",
    ]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
