"""In-tree build of the CUDA library (sm_100a only).

``python -m cudf_b200.build`` compiles cudf_b200/csrc/b2_groupby.cu into
cudf_b200/libb2groupby.so with nvcc.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc", "b2_groupby.cu")
DEPS = [SRC, os.path.join(HERE, "csrc", "b2_kernels.cuh"), os.path.join(HERE, "csrc", "b2_lean.cuh"), os.path.join(HERE, "csrc", "b2_partition.cuh"), os.path.join(HERE, "csrc", "b2_device.cuh"),
        os.path.join(os.path.dirname(HERE), "include", "b2_groupby.h")]
LIB = os.path.join(HERE, "libb2groupby.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared", "-cudart", "shared", "-ldl"]


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return nvcc


def stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(d) > t for d in DEPS)


def build(force: bool = False, verbose: bool = False) -> str:
    """Builds libb2groupby.so when it is missing or older than its sources; returns its path."""
    if not force and not stale():
        return LIB
    cmd = [find_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB, SRC]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
