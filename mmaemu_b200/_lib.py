"""ctypes binding of libmmaemu_b200.so (the C ABI declared in include/mmaemu_b200.h).

There is no fallback: if the shared object is missing or a call fails, an exception is raised
(BackendUnavailableError for a missing library or a device that is not sm_100).
"""
from __future__ import annotations

import ctypes
import threading
from pathlib import Path

from .errors import BackendUnavailableError

LIB_PATH = Path(__file__).resolve().parent / "libmmaemu_b200.so"
ABI_VERSION = 4

FMT_CODES = {"e4m3": 0, "e5m2": 1}
OUT_CODES = {"float32": 0, "bfloat16": 1, "float16": 2, "float8_e4m3fn": 3, "float8_e5m2": 4}
SCHEME_CODES = {"none": 0, "serial": 1, "pairwise": 2, "contiguous": 3}
KERNEL_CODES = {"auto": 0, "integer": 1, "fast": 2}
OK, ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_ARCH, ERR_LAUNCH, ERR_TOO_LARGE, ERR_TIMEOUT = 0, -1, -2, -3, -4, -5, -6

EXPORTS = ("mmb200_abi_version", "mmb200_status_string", "mmb200_last_cuda_error", "mmb200_device_supported",
           "mmb200_chain", "mmb200_accumulate", "mmb200_scaled_mm", "mmb200_scaled_mm_host", "mmb200_kernel_for",
           "mmb200_launch_count", "mmb200_workspace_bytes", "mmb200_workspace_bytes_split", "mmb200_scaled_mm_ws", "mmb200_accumulate_ws",
           "mmb200_scaled_mm_static", "mmb200_quantize_scaled_mm_ws", "mmb200_workspace_status_offset",
           "mmb200_workspace_status", "mmb200_scaled_mm_static_status", "mmb200_test_hooks", "mmb200_scaled_mm_peers", "mmb200_probe_issue_rate")

_lock = threading.Lock()
_lib = None


class NativeError(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, fn: str, status: int, text: str):
        super().__init__(f"{fn} failed with status {status}: {text}")
        self.status = status


def load():
    """The loaded library (loads it on first use). Raises BackendUnavailableError if it was never built."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not LIB_PATH.exists():
            raise BackendUnavailableError(
                f"{LIB_PATH} is missing: build it with `python -m mmaemu_b200.build` (needs nvcc); mmaemu_b200 has no "
                f"CPU or PyTorch fallback")
        try:
            L = ctypes.CDLL(str(LIB_PATH))
        except OSError as e:
            raise BackendUnavailableError(f"cannot load {LIB_PATH}: {e}") from e
        vp, i64, ci, cf = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
        L.mmb200_abi_version.argtypes = []
        L.mmb200_abi_version.restype = ci
        L.mmb200_status_string.argtypes = [ci]
        L.mmb200_status_string.restype = ctypes.c_char_p
        L.mmb200_last_cuda_error.argtypes = []
        L.mmb200_last_cuda_error.restype = ctypes.c_char_p
        L.mmb200_device_supported.argtypes = [ci]
        L.mmb200_device_supported.restype = ci
        L.mmb200_chain.argtypes = [vp, i64, ci, vp, i64, ci, vp, i64, ci, ci, ci, ci, ci, vp]
        L.mmb200_chain.restype = ci
        L.mmb200_accumulate.argtypes = [vp, i64, ci, vp, i64, ci, vp, i64, ci, ci, ci, ci, ci, ci, ci, ci, vp]
        L.mmb200_accumulate.restype = ci
        L.mmb200_scaled_mm.argtypes = [vp, i64, ci, vp, i64, ci, vp, i64, ci, ci, ci, ci, ci, ci, ci, ci, vp, vp, vp,
                                       ci, vp]
        L.mmb200_scaled_mm.restype = ci
        L.mmb200_scaled_mm_host.argtypes = [vp, i64, ci, vp, i64, ci, vp, i64, ci, ci, ci, ci, ci, ci, ci, ci, cf, cf,
                                            vp, ci, vp]
        L.mmb200_scaled_mm_host.restype = ci
        L.mmb200_workspace_bytes.argtypes = [ci, ci, ci]
        L.mmb200_workspace_bytes.restype = ctypes.c_size_t
        L.mmb200_workspace_bytes_split.argtypes = [ci, ci, ci, ci]
        L.mmb200_workspace_bytes_split.restype = ctypes.c_size_t
        L.mmb200_scaled_mm_ws.argtypes = [vp, i64, ci, vp, i64, ci, vp, i64, ci, ci, ci, ci, ci, ci, ci, ci, vp, vp, vp,
                                          ci, vp, ctypes.c_size_t, vp]
        L.mmb200_scaled_mm_ws.restype = ci
        L.mmb200_quantize_scaled_mm_ws.argtypes = [vp, i64, ci, vp, vp, i64, vp, i64, ci, vp, i64, ci, ci, ci, ci, ci, ci,
                                                   ci, ci, vp, vp, vp, vp, ctypes.c_size_t, vp]
        L.mmb200_quantize_scaled_mm_ws.restype = ci
        L.mmb200_accumulate_ws.argtypes = [vp, i64, ci, vp, i64, ci, vp, i64, ci, ci, ci, ci, ci, ci, ci, ci, vp,
                                           ctypes.c_size_t, vp]
        L.mmb200_accumulate_ws.restype = ci
        L.mmb200_scaled_mm_static.argtypes = [vp, i64, ci, vp, i64, ci, vp, i64, ci, ci, ci, ci, ci, ci, vp, vp, vp, vp]
        L.mmb200_scaled_mm_static.restype = ci
        L.mmb200_scaled_mm_peers.argtypes = [vp, i64, ci, vp, i64, ci, vp, i64, ci, ci, ci, ci, ci, ci, ci, ci, vp, vp, vp,
                                             ci, vp, ctypes.c_size_t, vp, ci, vp]
        L.mmb200_scaled_mm_peers.restype = ci
        L.mmb200_probe_issue_rate.argtypes = [ci, ci, ci, vp, vp]
        L.mmb200_probe_issue_rate.restype = ci
        L.mmb200_workspace_status_offset.argtypes = [ci, ci, ci, ci]
        L.mmb200_workspace_status_offset.restype = ctypes.c_size_t
        L.mmb200_workspace_status.argtypes = [vp, ci, ci, ci, ci, vp]
        L.mmb200_workspace_status.restype = ci
        L.mmb200_scaled_mm_static_status.argtypes = [ci, ci, ci, vp]
        L.mmb200_scaled_mm_static_status.restype = ci
        L.mmb200_test_hooks.argtypes = [ci, ci]
        L.mmb200_test_hooks.restype = None
        L.mmb200_kernel_for.argtypes = [vp, i64, vp, i64, ci, ci, ci]
        L.mmb200_kernel_for.restype = ci
        L.mmb200_launch_count.argtypes = []
        L.mmb200_launch_count.restype = i64
        got = L.mmb200_abi_version()
        if got != ABI_VERSION:
            raise BackendUnavailableError(f"{LIB_PATH} has ABI version {got}, this package needs {ABI_VERSION}; "
                                          f"rebuild it with `python -m mmaemu_b200.build --force`")
        _lib = L
        return _lib


def check(fn: str, status: int) -> None:
    """Raise for a negative status: BackendUnavailableError for a wrong device, NativeError otherwise."""
    if status == OK:
        return
    L = load()
    text = L.mmb200_status_string(status).decode()
    if status == ERR_LAUNCH:
        text += ": " + L.mmb200_last_cuda_error().decode()
    if status == ERR_ARCH:
        raise BackendUnavailableError(f"{fn}: {text}")
    raise NativeError(fn, status, text)


def launch_count() -> int:
    return int(load().mmb200_launch_count())
