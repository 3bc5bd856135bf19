"""Exception and warning classes, mirroring the reference's hierarchy class for class
(astding/mmaemu, mmaemu/errors.py:9-57) so that `except` clauses and exact-class checks written for the reference
keep working. When the reference package itself is importable its classes are re-used, so both packages raise the
very same types."""
from __future__ import annotations

__all__ = ["MmaemuError", "ReferenceRejectsError", "UnsupportedFeatureError", "SplitKUnknownError",
           "BackendUnavailableError", "ExperimentalPresetWarning", "UnverifiedSplitWarning",
           "UnvalidatedEnvelopeWarning", "BackendFallbackWarning"]

try:  # share the reference's classes when it is installed next to this package
    from mmaemu.errors import (BackendFallbackWarning, BackendUnavailableError, ExperimentalPresetWarning,  # noqa: F401
                               MmaemuError, ReferenceRejectsError, SplitKUnknownError, UnsupportedFeatureError,
                               UnvalidatedEnvelopeWarning, UnverifiedSplitWarning)
except Exception:  # noqa: BLE001 - standalone installation

    class MmaemuError(Exception):
        """Base class of every error of this package."""

    class ReferenceRejectsError(MmaemuError, RuntimeError):
        """The emulated platform (torch 2.7.1 or the profile's cuBLAS) rejects this call; raised where it does."""

    class UnsupportedFeatureError(MmaemuError, NotImplementedError):
        """Valid on the emulated platform but outside the modelled scope (bias, row-wise scales, autograd)."""

    class SplitKUnknownError(MmaemuError, LookupError):
        """The split-K decision of cuBLAS for this call is not known."""

    class BackendUnavailableError(MmaemuError, RuntimeError):
        """The CUDA backend cannot run here (library not built, no sm_100 device, CPU tensors)."""

    class ExperimentalPresetWarning(UserWarning):
        """The selected preset or profile is experimental."""

    class UnverifiedSplitWarning(UserWarning):
        """The split-K decision used was never replayed on hardware."""

    class UnvalidatedEnvelopeWarning(UnverifiedSplitWarning):
        """S = 1 was inferred by a split-K envelope that did not pass its held-out test."""

    class BackendFallbackWarning(RuntimeWarning):
        """Kept for interface parity; this package never falls back."""
