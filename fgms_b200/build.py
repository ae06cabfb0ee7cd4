"""Build ``libfgms_b200.so`` in-tree with nvcc for sm_100a.

    python -m fgms_b200.build [--force] [--verbose]

The library is a plain C-ABI shared object (see ``include/fgms_b200.h``); it links only the CUDA
runtime, not PyTorch.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libfgms_b200.so")
SOURCES = [os.path.join(CSRC, "fgms_abi.cu")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
"-Xcompiler", "-fPIC", "-shared", "-cudart", "shared", "-ldl",
]


def _deps():
    out = list(SOURCES)
    for d in (CSRC, os.path.join(os.path.dirname(HERE), "include")):
        out += [os.path.join(d, f) for f in os.listdir(d) if f.endswith((".cuh", ".h", ".cu"))]
    return out


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(f) > t for f in _deps())


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    extra = ["-DFGMS_NO_UMMA"] if os.environ.get("FGMS_NO_UMMA") == "1" else []  # bring-up aid only
    cmd = [nvcc] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + SOURCES + ["-o", LIB]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libfgms_b200.so")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
