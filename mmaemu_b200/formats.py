"""FP8 operand formats of the emulated tensor cores: torch dtype <-> format name, code classes, constants.

Mirrors the reference's format rules (astding/mmaemu, mmaemu/formats.py:14-62): only the OCP encodings NVIDIA tensor
cores implement are modelled -- E4M3 (torch.float8_e4m3fn: no Inf, NaN = S.1111.111) and E5M2 (torch.float8_e5m2:
Inf = S.11111.00, NaN = S.11111.{01,10,11}); the AMD fnuz encodings raise TypeError.
"""
from __future__ import annotations

import torch

E4M3, E5M2 = torch.float8_e4m3fn, torch.float8_e5m2
NAME_OF = {E4M3: "e4m3", E5M2: "e5m2"}
DTYPE_OF = {"e4m3": E4M3, "e5m2": E5M2}
FP8_MAX = {"e4m3": 448.0, "e5m2": 57344.0}
EMIN = {"e4m3": -6, "e5m2": -14}
MANT_BITS = {"e4m3": 3, "e5m2": 2}
CANONICAL_NAN_BITS = {torch.float32: 0x7FFFFFFF, torch.bfloat16: 0x7FFF, torch.float16: 0x7FFF, E4M3: 0x7F, E5M2: 0x7F}
OUT_DTYPE_NAMES = {torch.float32: "float32", torch.bfloat16: "bfloat16", torch.float16: "float16",
                   E4M3: "float8_e4m3fn", E5M2: "float8_e5m2"}
_FNUZ = tuple(getattr(torch, n) for n in ("float8_e4m3fnuz", "float8_e5m2fnuz") if hasattr(torch, n))


def is_fp8_dtype(dtype) -> bool:
    return dtype in NAME_OF


def fmt_of(dtype) -> str:
    """'e4m3' / 'e5m2' for the two modelled dtypes; TypeError otherwise (fnuz gets its own message)."""
    name = NAME_OF.get(dtype) if isinstance(dtype, torch.dtype) else None
    if name is not None:
        return name
    if dtype in _FNUZ:
        raise TypeError(f"{dtype} is an AMD fnuz encoding; NVIDIA tensor cores use float8_e4m3fn / float8_e5m2")
    raise TypeError(f"expected torch.float8_e4m3fn or torch.float8_e5m2, got {dtype}")


def nonfinite_mask(codes_u8: torch.Tensor, fmt: str) -> torch.Tensor:
    """True where a code is NaN (E4M3, E5M2) or Inf (E5M2)."""
    if fmt not in DTYPE_OF:
        raise ValueError(f"unknown FP8 format {fmt!r}")
    if codes_u8.dtype != torch.uint8:
        raise TypeError(f"codes must be uint8, got {codes_u8.dtype}")
    return (codes_u8 & 0x7F) == 0x7F if fmt == "e4m3" else (codes_u8 & 0x7C) == 0x7C
