"""The B200 kernels as a backend object of the reference's plugin interface.

The reference composes a GEMM from ChainFn calls -- `(a_u8 [M, L], b_u8 [N, L]) -> fp32 [M, N]`, one chain per output
from +0 over finite codes -- and picks who serves them through a Backend protocol: `name`, `supports(req)`,
`chain_fn(req)` (astding/mmaemu, mmaemu/backends/__init__.py:34-53; the wrapper every CUDA kernel shares is
mmaemu/backends/cuda/kernels.py:85-134). `B200Backend` implements that protocol on `mmb200_chain`, for every FP8
format pair and both characterised presets, so the reference's plan executor can run on it unchanged.
`install_into_reference()` makes `backend="cuda:b200"` (and "auto" / "cuda" on an sm_100 device) select it inside an
importable mmaemu package.

Argument errors follow the reference's wrapper: wrong dtypes raise TypeError; wrong ranks, mixed devices, K mismatch
and L % 16 != 0 raise ValueError before anything is launched. Launches go to torch's current stream of the tensors'
device. Operands may be views with storage offsets; they are made contiguous (a copy only when needed).
"""
from __future__ import annotations

import ctypes

from . import _lib
from .errors import BackendUnavailableError
from .numerics import get_preset

NAME = "cuda:b200"
K_MAX = 1 << 24


def _codes(t, name: str):
    import torch
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name}: expected a torch.Tensor, got {type(t).__name__}")
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        return t.view(torch.uint8)
    if t.dtype == torch.uint8:
        return t
    raise TypeError(f"{name}: the kernels take FP8 codes (torch.uint8, float8_e4m3fn or float8_e5m2), got {t.dtype}")


class B200Backend:
    """Backend protocol object; `kernel` picks the kernel family ('auto', 'integer', 'fast')."""

    def __init__(self, kernel: str = "auto"):
        if kernel not in _lib.KERNEL_CODES:
            raise ValueError(f"kernel must be one of {sorted(_lib.KERNEL_CODES)}, got {kernel!r}")
        self.kernel = kernel
        self.name = NAME if kernel == "auto" else f"{NAME}-{kernel}"

    def __repr__(self):
        return f"B200Backend(kernel={self.kernel!r})"

    def supports(self, req) -> str | None:
        """None if `req` (device, fmt_a, fmt_b, preset) can be served, else the reason."""
        import torch
        dev = torch.device(req.device)
        if dev.type != "cuda":
            return f"{self.name} needs a CUDA device, got {dev}"
        if req.fmt_a not in _lib.FMT_CODES or req.fmt_b not in _lib.FMT_CODES:
            return f"unknown FP8 formats {req.fmt_a!r} x {req.fmt_b!r}"
        try:
            preset = get_preset(req.preset)
        except Exception as e:  # noqa: BLE001
            return str(e)
        if preset.late_c and self.kernel == "fast":
            return f"preset {preset.name!r} (late accumulator, 25 fraction bits) is served by the integer kernel only"
        try:
            L = _lib.load()
        except BackendUnavailableError as e:
            return str(e)
        idx = dev.index if dev.index is not None else torch.cuda.current_device()
        if L.mmb200_device_supported(idx) != _lib.OK:
            return f"device {dev} is not sm_100 (the library holds sm_100a kernels only)"
        return None

    def chain_fn(self, req):
        import torch
        why = self.supports(req)
        if why is not None:
            raise BackendUnavailableError(why)
        device = torch.device(req.device)
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        fa, fb = _lib.FMT_CODES[req.fmt_a], _lib.FMT_CODES[req.fmt_b]
        nfma = get_preset(req.preset).code        # the preset's number at the C boundary
        kernel = _lib.KERNEL_CODES[self.kernel]
        L = _lib.load()
        name = self.name

        def chain(a, b):
            A, B = _codes(a, "a"), _codes(b, "b")
            if A.dim() != 2 or B.dim() != 2:
                raise ValueError(f"expected a [M, L] and b [N, L], got {tuple(A.shape)} and {tuple(B.shape)}")
            if A.device != device or B.device != device:
                raise ValueError(f"mixed devices: a on {A.device}, b on {B.device}, backend {name} on {device}")
            M, K = A.shape
            N, K2 = B.shape
            if K != K2:
                raise ValueError(f"K mismatch: a has {K}, b has {K2}")
            out = torch.empty((M, N), dtype=torch.float32, device=device)
            if M == 0 or N == 0:
                return out
            if K == 0:
                return out.zero_()
            if K % 16:
                raise ValueError(f"backend {name}: L = {K} is not a multiple of 16 (the plan zero-pads K)")
            if K >= K_MAX:
                raise ValueError(f"backend {name}: L = {K} >= {K_MAX}")
            A, B = A.contiguous(), B.contiguous()
            with torch.cuda.device(device):
                stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
                rc = L.mmb200_chain(A.data_ptr(), K, fa, B.data_ptr(), K, fb, out.data_ptr(), N, M, N, K, nfma, kernel,
                                    stream)
            _lib.check("mmb200_chain", rc)
            return out

        chain.backend = name
        return chain


BACKEND = B200Backend()


def install_into_reference():
    """Make an importable `mmaemu` package select this backend: backend='cuda:b200' always, and 'auto' / 'cuda' when
    the request's device is sm_100. Everything else falls through to the reference's own selection rules
    (mmaemu/backends/registry.py:194-267). `mmaemu.backends_status()` and `mmaemu.explain()` report the backend too.
    Errors are raised with the reference's own exception classes. Returns the patched registry module. Idempotent."""
    import importlib
    registry = importlib.import_module("mmaemu.backends.registry")
    if getattr(registry, "_mmaemu_b200_installed", False):
        return registry
    ref_errors = importlib.import_module("mmaemu.errors")
    backends = importlib.import_module("mmaemu.backends")
    original_select, original_explain, original_status = registry.select, registry.explain_selection, registry.status
    by_name = {NAME: BACKEND, f"{NAME}-integer": B200Backend("integer"), f"{NAME}-fast": B200Backend("fast")}

    def _choose(req, backend):
        """The B200 backend object for this request and backend name, or None to fall through."""
        import os
        name = backend
        if name == "auto":
            name = os.environ.get("MMAEMU_BACKEND", "").strip() or "auto"
        if name in by_name:
            be = by_name[name]
            why = be.supports(req)
            if why is not None:
                raise ref_errors.BackendUnavailableError(f"backend {name!r} cannot serve this call: {why}")
            return be
        if name in ("auto", "cuda") and BACKEND.supports(req) is None:
            return BACKEND
        return None

    def select(req, backend="auto"):
        be = _choose(req, backend)
        return be if be is not None else original_select(req, backend)

    def explain_selection(req, backend="auto"):
        be = _choose(req, backend)
        return (be, []) if be is not None else original_explain(req, backend)

    def status(device=None):
        import torch
        out = original_status(device)
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        dev = torch.device(device)
        req = backends.ChainRequest(device=dev, fmt_a="e4m3", fmt_b="e4m3", preset="hopper")
        why = BACKEND.supports(req)
        entry = backends.BackendStatus(name=NAME, available=why is None, source="precompiled sm_100a" if why is None else None,
                                       validated_here=why is None, reason=why or "")
        return {NAME: entry, **out}

    registry.select, registry.explain_selection, registry.status = select, explain_selection, status
    registry._mmaemu_b200_installed = True
    registry._mmaemu_b200_originals = (original_select, original_explain, original_status)
    if NAME not in backends.BACKEND_NAMES:
        backends.BACKEND_NAMES = tuple(backends.BACKEND_NAMES) + tuple(by_name)
    return registry


def uninstall_from_reference():
    """Undo install_into_reference (tests)."""
    import importlib
    registry = importlib.import_module("mmaemu.backends.registry")
    if not getattr(registry, "_mmaemu_b200_installed", False):
        return
    registry.select, registry.explain_selection, registry.status = registry._mmaemu_b200_originals
    registry._mmaemu_b200_installed = False
    backends = importlib.import_module("mmaemu.backends")
    backends.BACKEND_NAMES = tuple(n for n in backends.BACKEND_NAMES if not n.startswith(NAME))
