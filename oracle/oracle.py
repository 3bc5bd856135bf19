"""numpy/ctypes front end of the CPU oracle (oracle/mmaemu_oracle.c).

TEST INFRASTRUCTURE ONLY. Only the test-suite, the smoke run and the benchmark's CPU-baseline leg import this module;
nothing in the mmaemu_b200 package does. Parity is pinned: oracle/pin_against_reference.py checks the C code against
the reference's Python model and against the reference's golden vectors, and tests/golden holds the vectors that
travel.

The functions mirror the reference's entry points for the path:
  accumulate   mmaemu.accumulate / mmaemu.model.plan.execute_plan  (api.py:382-421, plan.py:169-208)
  scaled_mm    mmaemu.scaled_mm after validation                   (api.py:329-346)
  epilogue     mmaemu.model.epilogue.apply                         (epilogue.py:65-78)
  dot          mmaemu.model.dot                                    (chain.py:145-182)
Operands are uint8 code arrays: a [M, K], b [N, K] (= mat2.t() of the column-major [K, N] operand).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "_build" / "libmmaemu_oracle.so"

FMT = {"e4m3": 0, "e5m2": 1}
OUT = {"float32": 0, "bfloat16": 1, "float16": 2, "float8_e4m3fn": 3, "float8_e5m2": 4}
OUT_NP = {"float32": np.uint32, "bfloat16": np.uint16, "float16": np.uint16, "float8_e4m3fn": np.uint8,
          "float8_e5m2": np.uint8}
SCHEME = {"none": 0, "serial": 1, "pairwise": 2, "contiguous": 3}
NFMA = {"ada": 16, "hopper": 32, "b200_mma_sync": 288}    # preset code: products per block (+ 256: late accumulator)

_lib = None


def build(force: bool = False) -> Path:
    """Compile the oracle with gcc (oracle/Makefile) if the shared object is missing or older than its source."""
    src = HERE / "mmaemu_oracle.c"
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-s"], check=True)
    return LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(LIB_PATH))
        vp, i64, ci, cf = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
        L.oracle_accumulate.argtypes = [vp, i64, ci, vp, i64, ci, vp, i64, ci, ci, ci, ci, ci, ci, ci, ci]
        L.oracle_scaled_mm.argtypes = [vp, i64, ci, vp, i64, ci, vp, i64, ci, ci, ci, ci, ci, ci, ci, ci, cf, cf, vp,
                                       ci]
        L.oracle_epilogue.argtypes = [vp, vp, ci, i64, cf, cf, vp]
        L.oracle_dot.argtypes = [vp, ci, vp, ci, vp, vp, ci, ci, ci]
        for f in (L.oracle_accumulate, L.oracle_scaled_mm, L.oracle_epilogue, L.oracle_dot, L.oracle_num_threads):
            f.restype = ci
        _lib = L
    return _lib


def _codes(x, name):
    x = np.ascontiguousarray(x)
    if x.dtype != np.uint8 or x.ndim != 2:
        raise TypeError(f"{name} must be a 2-D uint8 code array")
    return x


def _nfma(preset):
    return NFMA[preset] if isinstance(preset, str) else int(preset)


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def accumulate(a, b, *, fmt_a="e4m3", fmt_b="e4m3", preset="hopper", fast=True, S=1, scheme="none",
               threads=0) -> np.ndarray:
    """fp32 accumulator bits (uint32 [M, N]) before alpha."""
    a, b = _codes(a, "a"), _codes(b, "b")
    M, K = a.shape
    N = b.shape[0]
    if b.shape[1] != K:
        raise ValueError("K mismatch")
    c = np.zeros((M, N), dtype=np.float32)
    rc = lib().oracle_accumulate(a.ctypes.data, max(K, 1), FMT[fmt_a], b.ctypes.data, max(K, 1), FMT[fmt_b],
                                 c.ctypes.data, max(N, 1), M, N, K, _nfma(preset), int(bool(fast)), int(S),
                                 SCHEME[scheme], int(threads))
    if rc:
        raise RuntimeError(f"oracle_accumulate failed ({rc})")
    return c.view(np.uint32)


def scaled_mm(a, b, scale_a, scale_b, *, out="bfloat16", fmt_a="e4m3", fmt_b="e4m3", preset="hopper", fast=False,
              S=1, scheme="none", scale_result=None, threads=0) -> np.ndarray:
    """Output bits ([M, N] of uint32 / uint16 / uint8 by out dtype) of the whole call."""
    a, b = _codes(a, "a"), _codes(b, "b")
    M, K = a.shape
    N = b.shape[0]
    if b.shape[1] != K:
        raise ValueError("K mismatch")
    d = np.zeros((M, N), dtype=OUT_NP[out])
    sr = None
    if scale_result is not None:
        sr = np.array([scale_result], dtype=np.float32)
    rc = lib().oracle_scaled_mm(a.ctypes.data, max(K, 1), FMT[fmt_a], b.ctypes.data, max(K, 1), FMT[fmt_b],
                                d.ctypes.data, max(N, 1), OUT[out], M, N, K, _nfma(preset), int(bool(fast)), int(S),
                                SCHEME[scheme], np.float32(scale_a), np.float32(scale_b),
                                sr.ctypes.data if sr is not None else None, int(threads))
    if rc:
        raise RuntimeError(f"oracle_scaled_mm failed ({rc})")
    return d


def epilogue(acc_bits, scale_a, scale_b, *, out="bfloat16", scale_result=None) -> np.ndarray:
    acc = np.ascontiguousarray(acc_bits).view(np.float32)
    d = np.zeros(acc.shape, dtype=OUT_NP[out])
    sr = None if scale_result is None else np.array([scale_result], dtype=np.float32)
    rc = lib().oracle_epilogue(acc.ctypes.data, d.ctypes.data, OUT[out], acc.size, np.float32(scale_a),
                               np.float32(scale_b), sr.ctypes.data if sr is not None else None)
    if rc:
        raise RuntimeError(f"oracle_epilogue failed ({rc})")
    return d


def dot(a, b, c=None, *, fmt_a="e4m3", fmt_b="e4m3", preset="ada") -> np.ndarray:
    """Instruction-level chains over the last dimension from c (fp32 bits as uint32, or None for +0)."""
    a, b = _codes(a, "a"), _codes(b, "b")
    rows, K = a.shape
    d = np.zeros(rows, dtype=np.float32)
    cc = None if c is None else np.ascontiguousarray(c).view(np.float32)
    rc = lib().oracle_dot(a.ctypes.data, FMT[fmt_a], b.ctypes.data, FMT[fmt_b],
                          cc.ctypes.data if cc is not None else None, d.ctypes.data, rows, K, _nfma(preset))
    if rc:
        raise RuntimeError(f"oracle_dot failed ({rc})")
    return d.view(np.uint32)


if __name__ == "__main__":
    print(build(force=bool(os.environ.get("FORCE"))))
