"""Builds libneura_cuda.so for sm_100a with nvcc, in-tree (neura_b200/lib/)."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "lib", "libneura_cuda.so")
SOURCES = ["neura_cuda.cu"]
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-shared",
]


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    inputs = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    inputs.append(os.path.join(HERE, "..", "include", "neura_cuda.h"))
    return any(os.path.getmtime(f) > built for f in inputs)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if a source is newer than it; returns its path."""
    if not (force or _stale()):
        return LIB
    os.makedirs(os.path.dirname(LIB), exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, *FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", LIB]
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
