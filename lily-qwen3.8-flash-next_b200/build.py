"""Builds the CUDA library in-tree with nvcc for sm_100a.

    python lily-qwen3.8-flash-next_b200/build.py [--force]

The result, liblily_sampler.so beside this file, exports the C ABI of
include/lily_sampler.h. nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB = os.path.join(HERE, "liblily_sampler.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def sources():
    out = []
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".cu", ".cpp")):
            out.append(os.path.join(CSRC, name))
    return out


def _deps():
    deps = [os.path.join(INCLUDE, n) for n in os.listdir(INCLUDE)]
    deps += [os.path.join(CSRC, n) for n in os.listdir(CSRC)]
    return deps


def stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(d) > t for d in _deps())


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not stale():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    extra = os.environ.get("LILY_NVCC_EXTRA", "").split()  # extra nvcc flags, e.g. -Xptxas -v
    cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", INCLUDE, "-o", LIB, *sources()]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        sys.stderr.write(proc.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
