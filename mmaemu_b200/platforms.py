"""Platform profiles: which GPU / cuBLASLt / caller a split-K decision and a hardware rejection refer to.

Host-side data, restating the reference's profile registry (astding/mmaemu, mmaemu/platform/profiles.py:76-235):
a profile pairs an instruction preset with the emulated platform's workspace size (which decides split-K), its
split-K table and the calls its cuBLASLt rejects. The six profiles of the scaled_mm path are provided, plus the two
without a platform, for which split-K can never be resolved automatically: `hopper-experimental` (hopper numerics)
and `b200-mma-sync-experimental` (the late-accumulator preset; unsplit fast accumulation only).

The emulated GPUs are an RTX 4060 and an H100 PCIe; a B200 is never one of them, so the reference's "live cuBLASLt
query on the profile's own GPU" step does not exist here (matches_device is always False).
"""
from __future__ import annotations

import os
from dataclasses import dataclass

DEFAULT_PROFILE = "hopper"


def _dtype_name(dt):
    if dt is None:
        return None
    s = str(dt)
    return s[6:] if s.startswith("torch.") else s


_FMT_ALIASES = {"float8_e4m3fn": "e4m3", "float8_e5m2": "e5m2"}


@dataclass(frozen=True)
class RejectRule:
    """A call the profile's cuBLASLt refuses. None matches anything; fmt_* are 'e4m3' / 'e5m2', out_dtype a torch
    dtype name."""
    fmt_a: str | None
    fmt_b: str | None
    out_dtype: str | None
    message: str

    def matches(self, fmt_a, fmt_b, out_dtype) -> bool:
        fa, fb = (_FMT_ALIASES.get(_dtype_name(x), _dtype_name(x)) for x in (fmt_a, fmt_b))
        od = _dtype_name(out_dtype)
        od = {"e4m3": "float8_e4m3fn", "e5m2": "float8_e5m2"}.get(od, od)
        return all(want is None or want == got for want, got in ((self.fmt_a, fa), (self.fmt_b, fb), (self.out_dtype, od)))


@dataclass(frozen=True)
class Profile:
    name: str
    preset: str
    gpu_name: str | None
    capability: tuple | None
    sm_count: int | None
    cublaslt_version: str | None
    caller: str
    torch_version: str | None
    workspace_bytes: int | None
    align: int | None
    splitk_table: str | None
    rejects: tuple
    maturity: str
    splitk_maturity: str
    description: str = ""

    def rejection(self, fmt_a, fmt_b, out_dtype):
        for r in self.rejects:
            if r.matches(fmt_a, fmt_b, out_dtype):
                return r
        return None

    def matches_device(self, device=None) -> bool:
        return False


def _reject(gpu: str) -> tuple:
    return (RejectRule("e4m3", "e4m3", "float8_e5m2",
                       f"cuBLASLt 12.8.3 on {gpu} rejects e4m3 x e4m3 -> e5m2 output (CUBLAS_STATUS_NOT_SUPPORTED); "
                       f"mixed e4m3/e5m2 inputs may produce e5m2"),)


_RTX4060 = dict(preset="ada", gpu_name="NVIDIA GeForce RTX 4060", capability=(8, 9), sm_count=24,
                cublaslt_version="12.8.3.14", torch_version="2.7.1+cu128", splitk_table="heur_rtx4060_lt12.8.3.14",
                rejects=_reject("sm_89"), maturity="validated")
_H100PCIE = dict(preset="hopper", gpu_name="NVIDIA H100 PCIe", capability=(9, 0), sm_count=114,
                 cublaslt_version="12.8.3.14", torch_version="2.7.1+cu128", splitk_table="heur_h100pcie_lt12.8.3.14",
                 rejects=_reject("the H100 (sm_90)"), maturity="validated")
_TORCH, _TE = "torch._scaled_mm", "transformer_engine"

PROFILES = {p.name: p for p in (
    Profile(name="ada", caller=_TORCH, workspace_bytes=1 << 20, align=None, splitk_maturity="validated",
            description="torch._scaled_mm on an RTX 4060 (24 SMs, cuBLASLt 12.8.3.14): 1 MiB workspace", **_RTX4060),
    Profile(name="ada-te", caller=_TE, workspace_bytes=4 << 20, align=256, splitk_maturity="experimental",
            description="Transformer Engine 2.3 on an RTX 4060: 4 MiB workspace; S > 1 decisions warn", **_RTX4060),
    Profile(name="ada-ws0", caller=_TORCH, workspace_bytes=0, align=None, splitk_maturity="validated",
            description="torch._scaled_mm on an RTX 4060 without a cuBLASLt workspace: never split", **_RTX4060),
    Profile(name="hopper", caller=_TORCH, workspace_bytes=1 << 20, align=None, splitk_maturity="validated",
            description="torch._scaled_mm on an H100 PCIe (114 SMs, cuBLASLt 12.8.3.14): 1 MiB workspace", **_H100PCIE),
    Profile(name="hopper-te", caller=_TE, workspace_bytes=32 << 20, align=256, splitk_maturity="experimental",
            description="Transformer Engine 2.3 on an H100 PCIe: 32 MiB workspace; S > 1 decisions and envelope "
                        "inferences warn", **_H100PCIE),
    Profile(name="hopper-ws0", caller=_TORCH, workspace_bytes=0, align=None, splitk_maturity="validated",
            description="torch._scaled_mm on an H100 PCIe without a cuBLASLt workspace: never split", **_H100PCIE),
    Profile(name="hopper-experimental", preset="hopper", gpu_name=None, capability=(9, 0), sm_count=None,
            cublaslt_version=None, caller=_TORCH, torch_version=None, workspace_bytes=None, align=None,
            splitk_table=None, rejects=(), maturity="experimental", splitk_maturity="none",
            description="hopper numerics without a reference platform (H100 SXM, H200, other cuBLASLt versions): no "
                        "split-K table, so splitk='auto' always raises SplitKUnknownError"),
    Profile(name="b200-mma-sync-experimental", preset="b200_mma_sync", gpu_name=None, capability=(10, 0),
            sm_count=None, cublaslt_version=None, caller=_TORCH, torch_version=None, workspace_bytes=None, align=None,
            splitk_table=None, rejects=(), maturity="experimental", splitk_maturity="none",
            description="fits the toolbox B200 mma.sync (HMMA-rewrite) vectors; NOT a model of sm_120 / RTX 5070 Ti; "
                        "NOT B200 cuBLAS; no split-K table: splitk='auto' always raises SplitKUnknownError"),
)}


def profile_maturity_warning(p: Profile, preset_validated: bool = True):
    """Warning text of an experimental profile whose preset is validated (an experimental preset warns by itself),
    else None (profiles.py:211-216)."""
    if p.maturity != "experimental" or not preset_validated:
        return None
    return f"profile {p.name!r} is experimental: {p.description}"


def list_profiles() -> list:
    return list(PROFILES)


def get_profile(name_or_profile=None) -> Profile:
    """Profile by name (None: $MMAEMU_PROFILE, else 'hopper'). A Profile object -- this package's, or any object with
    the same fields such as the reference's -- is accepted as is."""
    if isinstance(name_or_profile, Profile):
        return name_or_profile
    if name_or_profile is not None and not isinstance(name_or_profile, str):
        if all(hasattr(name_or_profile, f) for f in ("preset", "workspace_bytes", "splitk_table", "rejects")):
            return name_or_profile
        raise TypeError(f"profile must be a name or a Profile, got {type(name_or_profile).__name__}")
    name = name_or_profile if name_or_profile is not None else (os.environ.get("MMAEMU_PROFILE") or DEFAULT_PROFILE)
    try:
        return PROFILES[name]
    except KeyError:
        raise KeyError(f"unknown profile {name!r}; known: {', '.join(PROFILES)}") from None
