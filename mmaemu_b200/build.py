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
# translation units: (source, extra defines). kernel_fast.cu is compiled once per FP8 format pair, in parallel.
UNITS = (("api.cu", ()), ("kernel_integer.cu", ()), ("static_scratch.cu", ()),
         ("kernel_fast.cu", ("-DMMB_PART=0",)), ("kernel_fast.cu", ("-DMMB_PART=1",)),
         ("kernel_fast.cu", ("-DMMB_PART=2",)), ("kernel_fast.cu", ("-DMMB_PART=3",)))
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "--fmad=false", "-std=c++17",
              "-Xcompiler", "-fPIC"]
OBJ = PKG / "csrc" / "_obj"


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
    env = dict(os.environ)
    env.pop("CC", None)      # a CC without its support files in the environment must not leak into nvcc's host pass
    env.pop("CXX", None)
    OBJ.mkdir(exist_ok=True)
    nvcc = nvcc_path()
    # a unit is compiled again when its object is older than its source, a shared header or this file
    shared = [*CSRC.glob("*.cuh"), PKG.parent / "include" / "mmaemu_b200.h", Path(__file__)]
    newest_shared = max(d.stat().st_mtime for d in shared)
    jobs = []
    for i, (src, defines) in enumerate(UNITS):
        obj = OBJ / f"{Path(src).stem}_{i}.o"
        cmd = [nvcc, *NVCC_FLAGS, *defines, *(["-Xptxas", "-v"] if verbose else []), "-c", str(CSRC / src), "-o", str(obj)]
        fresh = (not force and not verbose and obj.exists()
                 and obj.stat().st_mtime > max(newest_shared, (CSRC / src).stat().st_mtime))
        proc = None if fresh else subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
        jobs.append((cmd, obj, proc))
    failed = None
    for cmd, obj, proc in jobs:
        if proc is None:
            continue
        out, _ = proc.communicate()
        if verbose or proc.returncode:
            sys.stderr.write(out)
        if proc.returncode and failed is None:
            failed = (proc.returncode, cmd)
    if failed:
        raise RuntimeError(f"nvcc failed ({failed[0]}): {' '.join(failed[1])}")
    cmd = [nvcc, "-shared", "-o", str(LIB), *[str(obj) for _, obj, _ in jobs]]
    r = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if verbose or r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode:
        raise RuntimeError(f"link failed ({r.returncode}): {' '.join(cmd)}")
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
