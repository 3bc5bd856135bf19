"""Builds libmmaemu_b200.so (the sm_100a kernels and their C ABI) in-tree with nvcc.

    python -m mmaemu_b200.build [--force] [--verbose]

The shared object sits next to this file, so it travels with a source checkout; it holds sm_100a code only.
Flags: --fmad=false (no contraction of the explicitly rounded fp32 operations), no fast-math, no flush-to-zero.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libmmaemu_b200.so"
SOURCES = ("api.cu", "kernel_integer.cu", "kernel_fast.cu", "static_scratch.cu")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "--fmad=false", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared"]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set $NVCC)")


def stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = [CSRC / s for s in SOURCES] + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "mmaemu_b200.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return LIB
    cmd = [nvcc_path(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", str(LIB),
           *[str(CSRC / s) for s in SOURCES]]
    env = dict(os.environ)
    env.pop("CC", None)      # a CC without its support files in the environment must not leak into nvcc's host pass
    env.pop("CXX", None)
    r = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if verbose or r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode:
        raise RuntimeError(f"nvcc failed ({r.returncode}): {' '.join(cmd)}")
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
