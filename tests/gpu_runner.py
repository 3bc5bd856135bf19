"""Runs numpy operands through the C ABI of libmmaemu_b200.so on cuda:0 and returns output bits (GPU tests only).

`scaled_mm` and `accumulate` take the same keyword arguments as the oracle's functions, so a test can feed one case to
both and compare. torch is used for device memory and the stream only."""
from __future__ import annotations

import ctypes

import os

import numpy as np
import torch

from mmaemu_b200 import _lib

OUT_NP = {"float32": np.uint32, "bfloat16": np.uint16, "float16": np.uint16, "float8_e4m3fn": np.uint8,
          "float8_e5m2": np.uint8}
OUT_TORCH = {"float32": torch.int32, "bfloat16": torch.int16, "float16": torch.int16, "float8_e4m3fn": torch.uint8,
             "float8_e5m2": torch.uint8}
DEV = torch.device("cuda:0")


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream(DEV).cuda_stream)


def _dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV)


def _ws(L, M, N, K, kernel, S=1):
    """Scratch memory for the staged kernels when `kernel` is 'staged', 'staged-whole', 'staged-int' or 'staged-rows'
    (test-side names: automatic choice + workspace; '-whole' turns K slicing off, so that few-tile shapes run the
    one-pass plan walkers; '-int' keeps the exponent pass of E4M3 x E4M3 on the CUDA cores instead of the tensor cores;
    '-rows' lets shapes with few output tiles run on the 16-row kernels, as the library does by default)."""
    os.environ["MMAEMU_B200_SLICES"] = "0" if kernel == "staged-whole" else "1"
    os.environ["MMAEMU_B200_TC_EPASS"] = "0" if kernel == "staged-int" else "1"
    # small shapes would all go to the 16-row kernels: only 'staged-rows' lets them ('staged*' otherwise keep the
    # 8-row-slot kernels under test; calls of at most 16 rows use the 16-row kernels either way)
    os.environ["MMAEMU_B200_ROW_GROUPS"] = "1" if kernel == "staged-rows" else "0"
    if kernel not in ("staged", "staged-whole", "staged-int", "staged-rows"):
        return None, None, 0, kernel
    n = int(L.mmb200_workspace_bytes_split(M, N, K, S))
    ws = torch.empty(max(n, 1), dtype=torch.uint8, device=DEV)
    return ws, ws.data_ptr(), n, "auto"


def _env_reset():
    """The launch has read the switches: later calls in this process (the Python entry points) see the defaults."""
    for name in ("MMAEMU_B200_SLICES", "MMAEMU_B200_TC_EPASS", "MMAEMU_B200_ROW_GROUPS"):
        os.environ.pop(name, None)


def scaled_mm(a, b, scale_a, scale_b, *, out="bfloat16", fmt_a="e4m3", fmt_b="e4m3", preset=32, fast=False, S=1,
              scheme="none", scale_result=None, kernel="auto", ld_pad=0):
    L = _lib.load()
    M, K = a.shape
    N = b.shape[0]
    if ld_pad:                                   # operands with a leading dimension larger than K
        a = np.concatenate([a, np.full((M, ld_pad), 0x55, np.uint8)], axis=1)
        b = np.concatenate([b, np.full((N, ld_pad), 0xAA, np.uint8)], axis=1)
    A, B = _dev(a), _dev(b)
    D = torch.full((M, max(N, 1)), -1 if OUT_TORCH[out] != torch.uint8 else 0xEE, dtype=OUT_TORCH[out], device=DEV)
    sc = torch.tensor([scale_a, scale_b, 1.0 if scale_result is None else scale_result], dtype=torch.float32,
                      device=DEV)
    ws, ws_ptr, ws_bytes, kernel = _ws(L, M, N, K, kernel, S)
    rc = L.mmb200_scaled_mm_ws(A.data_ptr(), K + ld_pad, _lib.FMT_CODES[fmt_a], B.data_ptr(), K + ld_pad,
                               _lib.FMT_CODES[fmt_b], D.data_ptr(), max(N, 1), _lib.OUT_CODES[out], M, N, K, int(preset),
                               int(bool(fast)), int(S), _lib.SCHEME_CODES[scheme], sc.data_ptr(), sc.data_ptr() + 4,
                               None if scale_result is None else sc.data_ptr() + 8, _lib.KERNEL_CODES[kernel], ws_ptr,
                               ws_bytes, _stream())
    _env_reset()
    _lib.check("mmb200_scaled_mm_ws", rc)
    torch.cuda.synchronize(DEV)
    return D[:, :N].cpu().numpy().view(OUT_NP[out])


def accumulate(a, b, *, fmt_a="e4m3", fmt_b="e4m3", preset=32, fast=True, S=1, scheme="none", kernel="auto"):
    L = _lib.load()
    M, K = a.shape
    N = b.shape[0]
    A, B = _dev(a), _dev(b)
    C = torch.full((M, max(N, 1)), -1, dtype=torch.int32, device=DEV)
    ws, ws_ptr, ws_bytes, kernel = _ws(L, M, N, K, kernel, S)
    rc = L.mmb200_accumulate_ws(A.data_ptr(), max(K, 1), _lib.FMT_CODES[fmt_a], B.data_ptr(), max(K, 1),
                                _lib.FMT_CODES[fmt_b], C.data_ptr(), max(N, 1), M, N, K, int(preset), int(bool(fast)),
                                int(S), _lib.SCHEME_CODES[scheme], _lib.KERNEL_CODES[kernel], ws_ptr, ws_bytes,
                                _stream())
    _env_reset()
    _lib.check("mmb200_accumulate_ws", rc)
    torch.cuda.synchronize(DEV)
    return C[:, :N].cpu().numpy().view(np.uint32)


def chain(a, b, *, fmt_a="e4m3", fmt_b="e4m3", preset=32, kernel="auto"):
    if kernel in ("staged", "staged-whole", "staged-int", "staged-rows"):     # the chain entry point has no workspace variant: fast plan, no patch
        clean = [np.where((x & 0x7F) == 0x7F, 0, x) if f == "e4m3" else np.where((x & 0x7C) == 0x7C, 0, x)
                 for x, f in ((a, fmt_a), (b, fmt_b))]
        return accumulate(clean[0].astype(np.uint8), clean[1].astype(np.uint8), fmt_a=fmt_a, fmt_b=fmt_b, preset=preset,
                          fast=True, kernel=kernel)
    L = _lib.load()
    M, K = a.shape
    N = b.shape[0]
    A, B = _dev(a), _dev(b)
    C = torch.full((M, N), -1, dtype=torch.int32, device=DEV)
    rc = L.mmb200_chain(A.data_ptr(), K, _lib.FMT_CODES[fmt_a], B.data_ptr(), K, _lib.FMT_CODES[fmt_b], C.data_ptr(),
                        N, M, N, K, int(preset), _lib.KERNEL_CODES[kernel], _stream())
    _lib.check("mmb200_chain", rc)
    torch.cuda.synchronize(DEV)
    return C.cpu().numpy().view(np.uint32)


def for_kernel(kernel):
    """(scaled_mm, accumulate) bound to one kernel family."""
    return (lambda *a, **k: scaled_mm(*a, kernel=kernel, **k)), (lambda *a, **k: accumulate(*a, kernel=kernel, **k))
