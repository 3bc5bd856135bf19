"""mmaemu_b200: the B200 (sm_100a) backend of mmaemu's scaled_mm path.

    import mmaemu_b200
    y = mmaemu_b200.scaled_mm(a_fp8, w_fp8.t(), scale_a, scale_b, out_dtype=torch.bfloat16, profile="hopper")

Same call signature, profiles, split-K resolution, exceptions and bits as mmaemu.scaled_mm; the computation runs in
hand-written sm_100a kernels behind a C ABI (include/mmaemu_b200.h, libmmaemu_b200.so). Importing the package does not
import torch or load the library; both happen on first use.
"""
from __future__ import annotations

import importlib

from .errors import (BackendFallbackWarning, BackendUnavailableError, ExperimentalPresetWarning, MmaemuError,  # noqa: F401
                     ReferenceRejectsError, SplitKUnknownError, UnsupportedFeatureError, UnvalidatedEnvelopeWarning,
                     UnverifiedSplitWarning)

__version__ = "0.1.0"

_LAZY = {
    "scaled_mm": ("mmaemu_b200.api", "scaled_mm"), "quantized_scaled_mm": ("mmaemu_b200.api", "quantized_scaled_mm"), "accumulate": ("mmaemu_b200.api", "accumulate"),
    "explain": ("mmaemu_b200.api", "explain"), "CallPlan": ("mmaemu_b200.api", "CallPlan"),
    "resolve_splitk": ("mmaemu_b200.splitk", "resolve_splitk"), "SplitK": ("mmaemu_b200.splitk", "SplitK"),
    "SplitDecision": ("mmaemu_b200.splitk", "SplitDecision"),
    "get_profile": ("mmaemu_b200.platforms", "get_profile"), "list_profiles": ("mmaemu_b200.platforms", "list_profiles"),
    "Profile": ("mmaemu_b200.platforms", "Profile"),
    "get_preset": ("mmaemu_b200.numerics", "get_preset"), "Preset": ("mmaemu_b200.numerics", "Preset"),
    "B200Backend": ("mmaemu_b200.backend", "B200Backend"), "BACKEND": ("mmaemu_b200.backend", "BACKEND"),
    "sharded_scaled_mm": ("mmaemu_b200.sharding", "sharded_scaled_mm"),
    "scaled_mm_into": ("mmaemu_b200.api", "scaled_mm_into"),
    "scaled_mm_host": ("mmaemu_b200.api", "scaled_mm_host"),
}

__all__ = ["__version__", *sorted(_LAZY), "MmaemuError", "ReferenceRejectsError", "UnsupportedFeatureError",
           "SplitKUnknownError", "BackendUnavailableError", "ExperimentalPresetWarning", "UnverifiedSplitWarning",
           "UnvalidatedEnvelopeWarning", "BackendFallbackWarning"]


def __getattr__(name: str):
    try:
        modname, attr = _LAZY[name]
    except KeyError:
        raise AttributeError(f"module 'mmaemu_b200' has no attribute {name!r}") from None
    value = getattr(importlib.import_module(modname), attr)
    globals()[name] = value
    return value


def __dir__():
    return sorted(set(globals()) | set(_LAZY))
