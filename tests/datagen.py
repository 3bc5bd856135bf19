"""Seeded operand generators shared by the tests: the data classes the reference's kernel conformance tests use
(astding/mmaemu, tests/test_kernels_ieee.py:44-92 and mmaemu/backends/cuda/selftest.py:42-81), written for numpy."""
from __future__ import annotations

import numpy as np

CLASSES = ("gauss1", "gauss40", "all_codes", "subnormal_zero", "max_mag", "block_exponents", "cancellation",
           "neg_zero")


def _finite(c, fmt):
    if fmt == "e4m3":
        return np.where((c & 0x7F) == 0x7F, c - 1, c).astype(np.uint8)
    return np.where((c & 0x7C) == 0x7C, c & 0x83, c).astype(np.uint8)


def _round_to(x, fmt):
    import torch
    dt = torch.float8_e4m3fn if fmt == "e4m3" else torch.float8_e5m2
    mx = 448.0 if fmt == "e4m3" else 57344.0
    return torch.from_numpy(np.clip(x, -mx, mx).astype(np.float32)).to(dt).view(torch.uint8).numpy().copy()


def codes(rng, rows, K, fmt, cls, side=0):
    """uint8 finite codes [rows, K] of one data class."""
    mb = 3 if fmt == "e4m3" else 2
    emax = 15 if fmt == "e4m3" else 30
    sign = (rng.random((rows, K)) < 0.5).astype(np.uint8) << 7
    man = rng.integers(0, 1 << mb, (rows, K), dtype=np.uint8)
    if cls == "gauss1":
        return _round_to(rng.standard_normal((rows, K)), fmt)
    if cls == "gauss40":
        return _round_to(rng.standard_normal((rows, K)) * 40, fmt)
    if cls == "all_codes":
        return _finite(rng.integers(0, 256, (rows, K), dtype=np.uint8), fmt)
    if cls == "subnormal_zero":                      # exponent field 0: subnormals and +-0
        return (sign | man).astype(np.uint8)
    if cls == "max_mag":                             # the largest finite codes: largest products and sums
        top = 0x7E if fmt == "e4m3" else 0x7B
        e = rng.integers(emax - 3, emax + 1, (rows, K), dtype=np.uint8)
        big = rng.random((rows, K)) < 0.6
        return _finite(np.where(big, sign | top, sign | (e << mb) | man).astype(np.uint8), fmt)
    if cls == "block_exponents":                     # one exponent per (row, 16-block)
        eb = rng.integers(0, emax + 1, (rows, (K + 15) // 16), dtype=np.uint8).repeat(16, axis=1)[:, :K]
        return _finite((sign | (eb << mb) | man).astype(np.uint8), fmt)
    if cls == "cancellation":                        # a[2j+1] = -a[2j] on side 0; b[2j+1] within one code of b[2j]
        c = _finite(rng.integers(0, 256, (rows, K), dtype=np.uint8), fmt)
        if side == 0:
            c[:, 1::2] = c[:, 0::2][:, :c[:, 1::2].shape[1]] ^ 0x80
        else:
            step = rng.integers(-1, 2, c[:, 1::2].shape)
            base = c[:, 0::2][:, :c[:, 1::2].shape[1]]
            top = 0x7E if fmt == "e4m3" else 0x7B
            c[:, 1::2] = (base & 0x80) | np.clip((base & 0x7F).astype(np.int16) + step, 0, top).astype(np.uint8)
        return c
    if cls == "neg_zero":
        c = _round_to(rng.standard_normal((rows, K)) * 4, fmt)
        return np.where(rng.random((rows, K)) < 0.3, np.uint8(0x80), c).astype(np.uint8)
    raise ValueError(cls)
