"""Public entry points: scaled_mm, accumulate, explain -- the reference's call signatures on the B200 kernels.

`scaled_mm` takes torch._scaled_mm's argument list (torch 2.7.1, `self` exposed as `input`) plus `profile=`,
`splitk=` and `backend=`, validates the call exactly as the reference does, resolves the split-K decision of the
emulated platform, and then makes ONE call into libmmaemu_b200.so that runs the accumulation plan, the non-finite
patch and the epilogue in a single kernel. There is no CPU path: CPU tensors raise BackendUnavailableError once the
call is otherwise valid.

Validation order (normative in the reference, astding/mmaemu mmaemu/api.py:8-23, 280-326; the exception classes and
the raise / no-raise outcome are what its parity tests pin):
  1. Python argument types                                   TypeError
  2. torch 2.7.1 _scaled_mm argument checks                  ReferenceRejectsError
     zero-size results return here (M or N == 0: empty; K == 0: +0), then the cuBLASLt checks: operand layouts,
     FP8 kinds, output dtype, 16-byte alignment, leading dimensions % 16
  3. profile rejects (e4m3 x e4m3 -> e5m2)                   ReferenceRejectsError
  4. scope: bias, row-wise scales, requires_grad             UnsupportedFeatureError
  5. maturity warning of the profile                         ExperimentalPresetWarning
  6. split-K resolution                                      SplitKUnknownError / ValueError
  7. backend: device and library                             BackendUnavailableError
"""
from __future__ import annotations

import ctypes
import os
import warnings
from dataclasses import dataclass, field

import torch

from . import _lib
from .errors import (BackendUnavailableError, ExperimentalPresetWarning, ReferenceRejectsError,
                     UnsupportedFeatureError)
from .formats import E4M3, E5M2, OUT_DTYPE_NAMES, fmt_of, is_fp8_dtype
from .numerics import check_plan, get_preset, maturity_warning, warn_once
from .platforms import get_profile, profile_maturity_warning
from .splitk import resolve_splitk

__all__ = ["scaled_mm", "scaled_mm_into", "accumulate", "explain", "CallPlan", "BACKEND_NAMES"]

BACKEND_NAMES = ("auto", "cuda", "cuda:b200", "cuda:b200-integer", "cuda:b200-fast", "cuda:b200-direct")
# kernel family behind each backend name; "direct" = automatic choice without scratch memory (operands are decoded
# inside the main loop instead of once into a workspace)
_KERNEL_OF = {"auto": "auto", "cuda": "auto", "cuda:b200": "auto", "cuda:b200-integer": "integer",
              "cuda:b200-fast": "fast", "cuda:b200-direct": "direct"}
# dtypes torch 2.7.1 lets through its "is a float8 matrix" check before the zero-size early return
_TORCH_FLOAT8 = {getattr(torch, n) for n in ("float8_e4m3fn", "float8_e5m2", "float8_e4m3fnuz", "float8_e5m2fnuz",
                                             "float8_e8m0fnu") if hasattr(torch, n)}


@dataclass
class CallPlan:
    """What a scaled_mm call would do (returned by explain)."""
    validation: object = "ok"            # "ok" or (error class name, message)
    profile: str = ""
    preset: str = ""
    preset_maturity: str = ""
    split: object = None                 # SplitDecision | None
    backend: str = ""
    fallbacks: list = field(default_factory=list)
    warnings: list = field(default_factory=list)


# ---------------------------------------------------------------------------------------------------------------
# layout predicates (as torch 2.7.1 hands matrices to cuBLASLt)
def _row_major(t) -> bool:
    return t.is_contiguous() or (t.stride(1) == 1 and t.stride(0) >= max(1, t.shape[1]))


def _col_major(t) -> bool:
    return not t.is_contiguous() and t.stride(0) == 1 and t.stride(1) >= max(1, t.shape[0])


def _misaligned(t) -> bool:
    if t.device.type == "cuda":
        return t.data_ptr() % 16 != 0
    return (t.storage_offset() * t.element_size()) % 16 != 0


# ---------------------------------------------------------------------------------------------------------------
def _check_argument_types(input, mat2, scale_a, scale_b, bias, scale_result, out_dtype, use_fast_accum, out):
    required = (("input", input), ("mat2", mat2), ("scale_a", scale_a), ("scale_b", scale_b))
    optional = (("bias", bias), ("scale_result", scale_result), ("out", out))
    for name, v in required:
        if not isinstance(v, torch.Tensor):
            raise TypeError(f"scaled_mm(): argument '{name}' must be Tensor, not {type(v).__name__}")
    for name, v in optional:
        if v is not None and not isinstance(v, torch.Tensor):
            raise TypeError(f"scaled_mm(): argument '{name}' must be Tensor, not {type(v).__name__}")
    if out_dtype is not None and not isinstance(out_dtype, torch.dtype):
        raise TypeError(f"scaled_mm(): argument 'out_dtype' must be torch.dtype, not {type(out_dtype).__name__}")
    if type(use_fast_accum) is not bool:
        raise TypeError(f"scaled_mm(): argument 'use_fast_accum' must be bool, not {type(use_fast_accum).__name__}")


def _check_like_torch(mat1, mat2, scale_a, scale_b, bias, scale_result, out_dtype, out):
    """The argument checks of torch 2.7.1's _scaled_mm_out_cuda, in its order. Returns (scaling kind, out dtype)."""
    def reject(msg):
        raise ReferenceRejectsError(msg)
    if mat1.dim() != 2:
        reject("mat1 must be a matrix")
    if mat2.dim() != 2:
        reject("mat2 must be a matrix")
    if mat1.shape[1] != mat2.shape[0]:
        reject(f"mat1 and mat2 shapes cannot be multiplied ({mat1.shape[0]}x{mat1.shape[1]} and "
               f"{mat2.shape[0]}x{mat2.shape[1]})")
    M, N = mat1.shape[0], mat2.shape[1]
    if scale_a.dtype != torch.float32 or scale_b.dtype != torch.float32:
        reject("Both scale_a and scale_b must be float (fp32) tensors.")
    if scale_a.numel() == 1 and scale_b.numel() == 1:
        scaling = "tensorwise"
    elif scale_a.dim() != 2 or scale_b.dim() != 2:
        reject("For non-TensorWise scaling, scale tensors must be 2-dimensional")
    elif tuple(scale_a.shape) == (M, 1) and tuple(scale_b.shape) == (1, N):
        if not (scale_a.is_contiguous() and scale_b.is_contiguous()):
            reject("Both scale_a and scale_b must be contiguous for RowWise scaling.")
        scaling = "rowwise"
    else:
        reject("Invalid scaling configuration. For TensorWise scaling, both scales should be scalar.")
    if scale_result is not None and (scale_result.numel() != 1 or scale_result.dtype != torch.float32):
        reject("scale_result must be a float scalar")
    if bias is not None and bias.numel() != N:
        reject(f"Bias must be size {N} but got {bias.numel()}")
    if mat1.shape[1] % 16:
        reject(f"Expected trailing dimension of mat1 to be divisible by 16 but got mat1 shape: "
               f"({mat1.shape[0]}x{mat1.shape[1]}).")
    if mat2.shape[0] % 16 or mat2.shape[1] % 16:
        reject(f"mat2 shape ({mat2.shape[0]}x{mat2.shape[1]}) must be divisible by 16")
    if out is not None and out_dtype is not None and out_dtype != out.dtype:
        reject("out_dtype must match output matrix type")
    od = out_dtype if out_dtype is not None else (out.dtype if out is not None else mat1.dtype)
    for name, t in (("mat1", mat1), ("mat2", mat2)):
        if t.dtype not in _TORCH_FLOAT8:
            reject(f"Expected {name} to be Float8 matrix got {t.dtype}")
    if mat1.dtype == E5M2 and mat2.dtype == E5M2:
        reject("Multiplication of two Float8_e5m2 matrices is not supported")
    if bias is not None:
        if od == torch.float32:
            reject("Bias is not supported when out_dtype is set to Float32")
        if bias.dtype not in (torch.bfloat16, torch.float16):
            reject(f"Bias must be either Half or BFloat16, but got {bias.dtype}")
        if od in (torch.bfloat16, torch.float16) and bias.dtype != od:
            reject(f"Bias must be {od} to compute {od} output, but got {bias.dtype}")
    for t in (out, mat2, bias, scale_a, scale_b, scale_result):
        if t is not None and t.device != mat1.device:
            reject(f"Expected all tensors to be on the same device, but found at least two devices, {mat1.device} and "
                   f"{t.device}!")
    return scaling, od


def _check_like_cublas(mat1, mat2, scaling, od):
    """Checks that apply to non-empty calls only. Returns mat1 as cuBLAS reads it (torch copies a mat1 that is neither
    row- nor column-major to a contiguous one)."""
    def reject(msg):
        raise ReferenceRejectsError(msg)
    if scaling == "rowwise" and od != torch.bfloat16:
        reject("Only bf16 high precision output types are supported for row-wise scaling.")
    if _col_major(mat1) or not _row_major(mat2.t()):
        reject("Only multiplication of row-major and column-major matrices is supported by cuBLASLt")
    if not _row_major(mat1):
        mat1 = mat1.contiguous()
    for name, t in (("mat1", mat1), ("mat2", mat2)):
        if not is_fp8_dtype(t.dtype):
            reject(f"{name} is {t.dtype}: torch 2.7.1 fails on CUDA for FP8 formats other than float8_e4m3fn and "
                   f"float8_e5m2")
    if od not in OUT_DTYPE_NAMES:
        reject(f"out dtype {od} is not supported by cuBLASLt FP8 GEMMs (CUBLAS_STATUS_NOT_SUPPORTED)")
    if _misaligned(mat1) or _misaligned(mat2):
        reject("CUBLAS_STATUS_NOT_SUPPORTED when calling cublasLtMatmul (operand pointer not 16-byte aligned)")
    lda = mat1.stride(0) if mat1.shape[0] > 1 else mat1.shape[1]
    ldb = mat2.stride(1) if mat2.shape[1] > 1 else mat2.shape[0]
    if lda % 16 or ldb % 16:
        reject("CUBLAS_STATUS_NOT_SUPPORTED when calling cublasLtMatmulAlgoGetHeuristic (leading dimension not a "
               "multiple of 16)")
    return mat1


def _check_scope(scaling, bias, tensors):
    if bias is not None:
        raise UnsupportedFeatureError("bias is not supported (cuBLAS's fused-bias epilogue is not modelled); add the "
                                      "bias yourself after scaled_mm")
    if scaling == "rowwise":
        raise UnsupportedFeatureError("row-wise scales are not supported (they run through a stream-K kernel whose "
                                      "split depends on the SM count)")
    if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors):
        raise UnsupportedFeatureError("inference only: an input requires grad while grad mode is enabled (use "
                                      "torch.no_grad() or detach the inputs)")


def _kernel_choice(backend: str) -> str:
    """'auto' | 'integer' | 'fast' for a backend name; BackendUnavailableError for the reference's own backends."""
    if not isinstance(backend, str):
        raise TypeError(f"backend must be a str, got {type(backend).__name__}")
    if backend == "auto":
        backend = os.environ.get("MMAEMU_BACKEND", "").strip() or "auto"
    if backend in _KERNEL_OF:
        return _KERNEL_OF[backend]
    if backend == "reference" or backend.startswith("cuda:"):
        raise BackendUnavailableError(f"backend {backend!r} is not part of mmaemu_b200 (available: "
                                      f"{', '.join(BACKEND_NAMES)}); the float64 reference model and the NVRTC kernels "
                                      f"live in the mmaemu package")
    raise ValueError(f"unknown backend {backend!r}; expected one of {', '.join(BACKEND_NAMES)}")


def _require_device(device: torch.device) -> None:
    if device.type != "cuda":
        raise BackendUnavailableError(f"mmaemu_b200 runs on sm_100 CUDA devices only and has no CPU fallback; got "
                                      f"tensors on {device}")
    L = _lib.load()
    idx = device.index if device.index is not None else torch.cuda.current_device()
    _lib.check("mmb200_device_supported", L.mmb200_device_supported(idx))


# ---------------------------------------------------------------------------------------------------------------
class _Call:
    """A validated call: shapes, formats, profile, split decision, kernel choice."""
    __slots__ = ("early", "unchanged_out", "M", "N", "K", "fa", "fb", "od", "profile", "preset", "decision", "scheme",
                 "kernel", "mat1", "notes")


def _maturity_message(prof, preset):
    """The maturity warning of the call: the preset's, else the profile's (mmaemu/api.py:121-124)."""
    return maturity_warning(preset) or profile_maturity_warning(prof, preset.maturity == "validated")


def _emit_maturity(prof, preset) -> None:
    """ExperimentalPresetWarning of the preset (once per name) or of the profile (once per name), as
    mmaemu/api.py:127-133."""
    msg = maturity_warning(preset)
    if msg is not None:
        warn_once(preset.name, msg, stacklevel=6)
    msg = profile_maturity_warning(prof, preset.maturity == "validated")
    if msg is not None:
        warn_once("profile:" + prof.name, msg, stacklevel=6)


def _prepare(input, mat2, scale_a, scale_b, bias, scale_result, out_dtype, use_fast_accum, out, profile, splitk,
             backend, *, dry: bool) -> _Call:
    c = _Call()
    c.notes = []
    _check_argument_types(input, mat2, scale_a, scale_b, bias, scale_result, out_dtype, use_fast_accum, out)
    scaling, c.od = _check_like_torch(input, mat2, scale_a, scale_b, bias, scale_result, out_dtype, out)
    c.M, c.K, c.N = input.shape[0], input.shape[1], mat2.shape[1]
    c.profile = get_profile(profile)
    c.preset = get_preset(c.profile.preset)
    c.early = c.M == 0 or c.N == 0 or c.K == 0
    c.unchanged_out = False
    c.decision = c.kernel = c.fa = c.fb = None
    c.scheme = "none"
    c.mat1 = input
    if c.early:
        return c
    c.mat1 = _check_like_cublas(input, mat2, scaling, c.od)
    c.fa, c.fb = fmt_of(c.mat1.dtype), fmt_of(mat2.dtype)
    rule = c.profile.rejection(c.fa, c.fb, c.od)
    if rule is not None:
        raise ReferenceRejectsError(f"{rule.message} [profile {c.profile.name}]")
    _check_scope(scaling, bias, (c.mat1, mat2, scale_a, scale_b, scale_result, bias))
    msg = _maturity_message(c.profile, c.preset)
    if msg is not None:
        c.notes.append(msg)
    if not dry:
        _emit_maturity(c.profile, c.preset)
    same_shape = out is not None and tuple(out.shape) == (c.M, c.N)
    if same_shape and not (_row_major(out) or _col_major(out)):
        # torch computes into a contiguous copy of such an out= and never copies the result back
        c.unchanged_out = True
        c.notes.append(f"out= with strides {tuple(out.stride())} is neither row- nor column-major: torch 2.7.1 computes "
                       f"into a contiguous copy and never copies it back, so out= is returned unchanged")
        return c
    layout_std = c.mat1.is_contiguous() and mat2.t().is_contiguous()
    if same_shape and _col_major(out):
        # a column-major out= is computed as the transposed problem with the formats swapped
        key = (c.N, c.M, c.K, mat2.dtype, c.mat1.dtype)
    else:
        key = (c.M, c.N, c.K, c.mat1.dtype, mat2.dtype)
    c.decision = resolve_splitk(key[0], key[1], key[2], a_dtype=key[3], b_dtype=key[4], out_dtype=c.od,
                                use_fast_accum=bool(use_fast_accum), profile=c.profile, splitk=splitk,
                                layout_std=layout_std, dry=dry)
    c.kernel = _kernel_choice(backend)
    if not dry:
        _require_device(c.mat1.device)
    return c


def _stream_ptr(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _scalar_ptr(t: torch.Tensor, device) -> tuple:
    """(keep-alive tensor, device pointer) of a one-element fp32 tensor on `device`."""
    t = t.detach()
    if t.device != device or not t.is_contiguous():
        t = t.to(device).contiguous()
    return t, t.data_ptr()


SPLIT_WORKSPACE_LIMIT = 8 << 30


def _workspace(L, kernel: str, a_ptr, lda, b_ptr, ldb, M, N, K, nfma, S, device):
    """(keep-alive tensor or None, pointer or None, bytes) of the scratch memory for the staged fast kernel. The tensor
    comes from torch's caching allocator, which hands it out again only to later work on the same stream."""
    if kernel in ("integer", "direct") or os.environ.get("MMAEMU_B200_WORKSPACE", "1") == "0":
        return None, None, 0
    if L.mmb200_kernel_for(a_ptr, lda, b_ptr, ldb, K, nfma, 1) != _lib.KERNEL_CODES["fast"]:
        return None, None, 0                 # operands the fast kernels cannot read: the integer kernel serves the call
    n = int(L.mmb200_workspace_bytes_split(M, N, K, S))
    if S > 1 and n > SPLIT_WORKSPACE_LIMIT:
        return None, None, 0                 # split plans keep 8 bytes of scratch per output; very large ones run on the integer kernel
    ws = torch.empty(n, dtype=torch.uint8, device=device)
    return ws, ws.data_ptr(), n


def _kernel_code(kernel: str) -> int:
    return _lib.KERNEL_CODES["auto" if kernel == "direct" else kernel]


def _run_scaled_mm(c: _Call, mat2, scale_a, scale_b, scale_result, fast: bool, y=None, peers=()) -> torch.Tensor:
    """The one call into the library. y: where the result goes (default: a new [M, N] tensor): row-major with unit
    stride along N. peers: device pointers, valid in this process, that receive the same elements at the same indices
    (the same [M, N] rectangle of other GPUs' result buffers)."""
    dev = c.mat1.device
    a = c.mat1.detach()
    bt = mat2.detach().t()                               # [N, K] with unit stride along K
    lda = a.stride(0) if c.M > 1 else c.K
    ldb = bt.stride(0) if c.N > 1 else c.K
    if y is None:
        y = torch.empty((c.M, c.N), dtype=c.od, device=dev)
    ldd = y.stride(0) if c.M > 1 else c.N
    keep_a, pa = _scalar_ptr(scale_a, dev)
    keep_b, pb = _scalar_ptr(scale_b, dev)
    keep_r, pr = (None, None) if scale_result is None else _scalar_ptr(scale_result, dev)
    L = _lib.load()
    peer_array = (ctypes.c_void_p * max(len(peers), 1))(*[ctypes.c_void_p(int(p)) for p in peers])
    with torch.cuda.device(dev):
        ws, ws_ptr, ws_bytes = _workspace(L, c.kernel, a.data_ptr(), lda, bt.data_ptr(), ldb, c.M, c.N, c.K,
                                          c.preset.code, c.decision.S, dev)
        rc = L.mmb200_scaled_mm_peers(a.data_ptr(), lda, _lib.FMT_CODES[c.fa], bt.data_ptr(), ldb,
                                      _lib.FMT_CODES[c.fb], y.data_ptr(), ldd, _lib.OUT_CODES[OUT_DTYPE_NAMES[c.od]],
                                      c.M, c.N, c.K, c.preset.code, int(fast), c.decision.S,
                                      _lib.SCHEME_CODES[c.scheme], pa, pb, pr, _kernel_code(c.kernel), ws_ptr, ws_bytes,
                                      peer_array, len(peers), _stream_ptr(dev))
    _lib.check("mmb200_scaled_mm_peers", rc)
    if ws is not None and os.environ.get("MMAEMU_B200_CHECK_STATUS", "0") == "1":
        # opt-in: wait for the call and read the status word of its bounded waits (a host synchronisation per call)
        with torch.cuda.device(dev):
            _lib.check("mmb200_workspace_status", L.mmb200_workspace_status(ws_ptr, c.M, c.N, c.K, c.decision.S,
                                                                            _stream_ptr(dev)))
    del keep_a, keep_b, keep_r, ws
    return y


def scaled_mm_into(y, peers, input, mat2, scale_a, scale_b, scale_result=None, use_fast_accum=False, *, profile=None,
                   splitk="auto", backend="auto"):
    """scaled_mm whose result is written into `y` -- an [M, N] row-major tensor or view (unit stride along N; any row
    stride, so a rectangle of a larger result works) -- and, element for element, into the memory at every device
    pointer of `peers` (the same rectangle of other GPUs' result buffers, mapped into this process). The building
    block of sharded_scaled_mm's fused assembly. Every check and raise is scaled_mm's, with out_dtype = y.dtype."""
    if not isinstance(y, torch.Tensor) or y.dim() != 2 or (y.shape[1] > 1 and y.stride(1) != 1):
        raise TypeError("scaled_mm_into(): y must be a 2-D tensor with unit stride along its last dimension")
    c = _prepare(input, mat2, scale_a, scale_b, None, scale_result, y.dtype, use_fast_accum, None, profile, splitk,
                 backend, dry=False)
    if tuple(y.shape) != (c.M, c.N):
        raise ValueError(f"scaled_mm_into(): y has shape {tuple(y.shape)}, the result is {(c.M, c.N)}")
    if y.device != input.device:
        raise ValueError(f"scaled_mm_into(): y is on {y.device}, the operands on {input.device}")
    if c.M == 0 or c.N == 0:
        return y
    if c.early:                                          # K == 0: +0 everywhere; peers are written by their own ranks' calls
        y.zero_()
        if peers:
            raise ValueError("scaled_mm_into(): K == 0 with peer buffers is not supported")
        return y
    c.scheme = check_plan(c.preset, c.K, c.decision.S, c.decision.scheme, bool(use_fast_accum))
    return _run_scaled_mm(c, mat2, scale_a, scale_b, scale_result, bool(use_fast_accum), y=y, peers=tuple(peers))


def scaled_mm(input, mat2, scale_a, scale_b, bias=None, scale_result=None, out_dtype=None, use_fast_accum=False,
              *, out=None, profile=None, splitk="auto", backend="auto"):
    """torch._scaled_mm with the numerics of the profile's GPU, computed by the B200 kernels.

    input [M, K] FP8 row-major; mat2 [K, N] FP8 column-major (e.g. w.t() of a row-major [N, K] weight); scale_a,
    scale_b: one-element fp32 tensors. Returns [M, N] of out_dtype (default input.dtype) on input.device, which must
    be an sm_100 CUDA device. profile: one of hopper (default, or $MMAEMU_PROFILE), hopper-te, hopper-ws0, ada,
    ada-te, ada-ws0. splitk: "auto", 1, a SplitK or (S, scheme). backend: "auto" | "cuda" | "cuda:b200" |
    "cuda:b200-integer" | "cuda:b200-fast". Raises what the reference raises (module docstring)."""
    c = _prepare(input, mat2, scale_a, scale_b, bias, scale_result, out_dtype, use_fast_accum, out, profile, splitk,
                 backend, dry=False)
    if c.unchanged_out:
        warnings.warn(c.notes[-1], UserWarning, stacklevel=2)
        return out
    if c.early:
        y = torch.zeros(c.M, c.N, dtype=c.od, device=input.device)
    else:
        c.scheme = check_plan(c.preset, c.K, c.decision.S, c.decision.scheme, bool(use_fast_accum))
        y = _run_scaled_mm(c, mat2, scale_a, scale_b, scale_result, bool(use_fast_accum))
    if out is None:
        return y
    if tuple(out.shape) != (c.M, c.N):
        if out.numel() != 0:
            warnings.warn(f"An output with one or more elements was resized since it had shape {list(out.shape)}, "
                          f"which does not match the required output shape {[c.M, c.N]}.", UserWarning, stacklevel=2)
        out.resize_(c.M, c.N)
    out.copy_(y)
    return out


def scaled_mm_host(input, mat2, scale_a, scale_b, scale_result=None, out_dtype=None, use_fast_accum=False, *, out=None,
                   profile=None, splitk="auto", backend="auto", device=None):
    """scaled_mm for operands that live in HOST memory: CPU tensors in, a CPU tensor out, computed on `device` (default:
    the current CUDA device) by the library's host-buffer entry point (mmb200_scaled_mm_host), which stages the operands
    on the device, overlaps the copies with the kernels slab by slab for large calls, and waits for the result.

    Arguments, checks, exceptions and their order are those of scaled_mm (the call is validated from the tensors'
    metadata). input [M, K] and mat2 [K, N] (column-major) are FP8 CPU tensors, pinned for full copy speed; the scales
    are one-element fp32 tensors. out: optional row-major [M, N] CPU tensor of the output dtype to write into (a new
    pinned tensor otherwise). The result equals scaled_mm on the same operands bit for bit."""
    from .sharding import validate_full_call
    for name, t in (("input", input), ("mat2", mat2)):
        if isinstance(t, torch.Tensor) and t.device.type != "cpu":
            raise ValueError(f"scaled_mm_host(): {name} is on {t.device}; this entry point takes host tensors "
                             f"(use scaled_mm for device tensors)")
    c = validate_full_call(input, mat2, scale_a, scale_b, None, scale_result, out_dtype, use_fast_accum, profile, splitk,
                           backend)
    if out is not None:
        if not isinstance(out, torch.Tensor) or out.device.type != "cpu" or out.dtype != c.od or \
                tuple(out.shape) != (c.M, c.N) or (c.N > 1 and out.stride(1) != 1) or (c.M > 1 and out.stride(0) < c.N):
            raise ValueError(f"scaled_mm_host(): out must be a row-major CPU tensor of shape {(c.M, c.N)} and dtype {c.od}")
    if c.early:
        y = out if out is not None else torch.empty((c.M, c.N), dtype=c.od)
        return y.zero_()
    fast = bool(use_fast_accum)
    scheme = check_plan(c.preset, c.K, c.decision.S, c.decision.scheme, fast)
    _emit_maturity(c.profile, c.preset)
    if not torch.cuda.is_available():
        raise BackendUnavailableError("mmaemu_b200 runs on sm_100 CUDA devices only and has no CPU fallback; no CUDA "
                                      "device is available to scaled_mm_host()")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if dev.type == "cuda" and dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    _require_device(dev)
    a = input.detach()
    bt = mat2.detach().t()                               # [N, K] with unit stride along K
    if a.stride(1) != 1 and c.K > 1:
        a = a.contiguous()
    lda = a.stride(0) if c.M > 1 else c.K
    ldb = bt.stride(0) if c.N > 1 else c.K
    y = out if out is not None else torch.empty((c.M, c.N), dtype=c.od, pin_memory=True)
    ldd = y.stride(0) if c.M > 1 else c.N
    sr = None if scale_result is None else ctypes.c_float(float(scale_result.detach().reshape(()).item()))
    L = _lib.load()
    with torch.cuda.device(dev):
        rc = L.mmb200_scaled_mm_host(a.data_ptr(), lda, _lib.FMT_CODES[c.fa], bt.data_ptr(), ldb, _lib.FMT_CODES[c.fb],
                                     y.data_ptr(), ldd, _lib.OUT_CODES[OUT_DTYPE_NAMES[c.od]], c.M, c.N, c.K,
                                     c.preset.code, int(fast), c.decision.S, _lib.SCHEME_CODES[scheme],
                                     ctypes.c_float(float(scale_a.detach().reshape(()).item())),
                                     ctypes.c_float(float(scale_b.detach().reshape(()).item())),
                                     None if sr is None else ctypes.cast(ctypes.pointer(sr), ctypes.c_void_p),
                                     _kernel_code(c.kernel), _stream_ptr(dev))
    _lib.check("mmb200_scaled_mm_host", rc)
    return y


def quantized_scaled_mm(x, quant_scale, mat2, scale_a, scale_b, scale_result=None, out_dtype=None,
                        use_fast_accum=False, *, profile=None, splitk="auto", return_codes=False):
    """scaled_mm on activations that are still in fp32 or bf16: the quantisation to E4M3,

        xq = (x * quant_scale).clamp(-448, 448).to(torch.float8_e4m3fn)          # as torch computes it on a CUDA device
        y  = scaled_mm(xq, mat2, scale_a, scale_b, ...)

    runs inside the pass that decodes the first operand instead of as separate torch operations (the recipe of the
    reference's FP8 examples, examples/evo2_offload.py:124-129 of astding/mmaemu: quant_scale = 448 / amax and
    scale_a = 1 / quant_scale). x: [M, K] fp32 or bf16, unit stride along K; quant_scale: one-element fp32 tensor
    (with bf16 activations torch's type promotion rounds it to bf16 before the multiplication, and so does this call).
    Everything else, including every check and raise, is scaled_mm's, applied to the E4M3 tensor the call produces.
    Returns y, or (y, xq) with return_codes=True. Activations or weights that the decode pass cannot read with 16-byte
    loads raise ValueError (there is no path through torch operations)."""
    if not isinstance(x, torch.Tensor) or x.dtype not in (torch.float32, torch.bfloat16) or x.dim() != 2:
        raise TypeError("quantized_scaled_mm(): x must be a 2-D fp32 or bf16 tensor")
    if not isinstance(quant_scale, torch.Tensor) or quant_scale.numel() != 1 or quant_scale.dtype != torch.float32:
        raise TypeError("quantized_scaled_mm(): quant_scale must be a one-element fp32 tensor")
    if torch.is_grad_enabled() and x.requires_grad:
        raise UnsupportedFeatureError("inference only: an input requires grad while grad mode is enabled")
    M, K = x.shape
    xq = torch.empty((M, K), dtype=torch.float8_e4m3fn, device=x.device)
    c = _prepare(xq, mat2, scale_a, scale_b, None, scale_result, out_dtype, use_fast_accum, None, profile, splitk,
                 "auto", dry=False)
    xs = x.detach()
    per16 = 4 if xs.dtype == torch.float32 else 8
    fused = (not c.early and K % 16 == 0 and xs.stride(1) == 1 and xs.stride(0) % per16 == 0
             and xs.data_ptr() % 16 == 0 and os.environ.get("MMAEMU_B200_WORKSPACE", "1") != "0")
    L = _lib.load() if fused else None
    if fused:
        c.scheme = check_plan(c.preset, c.K, c.decision.S, c.decision.scheme, bool(use_fast_accum))
        if c.preset.late_c:
            raise UnsupportedFeatureError(f"quantized_scaled_mm(): preset {c.preset.name!r} runs on the integer kernel, "
                                          f"which has no quantisation pass; quantise with torch and call scaled_mm")
        dev = x.device
        bt = mat2.detach().t()
        ldb = bt.stride(0) if c.N > 1 else c.K
        fused = bt.data_ptr() % 16 == 0 and ldb % 16 == 0
    if not fused and not c.early:
        raise ValueError("quantized_scaled_mm(): the quantisation runs inside the kernels' decode pass, which reads x and "
                         "mat2 with 16-byte loads and needs scratch memory: x must have unit stride along K, 16-byte "
                         "aligned rows (base address and row stride), mat2.t() must be 16-byte aligned with a leading "
                         "dimension that is a multiple of 16, and MMAEMU_B200_WORKSPACE must not be 0. Quantise with "
                         "torch and call scaled_mm for other layouts.")
    if c.early:
        y = scaled_mm(xq, mat2, scale_a, scale_b, None, scale_result, out_dtype, use_fast_accum, profile=profile,
                      splitk=splitk)                     # zero-size result: nothing to quantise or compute
        return (y, xq) if return_codes else y
    y = torch.empty((c.M, c.N), dtype=c.od, device=dev)
    keep_q, pq = _scalar_ptr(quant_scale, dev)
    keep_a, pa = _scalar_ptr(scale_a, dev)
    keep_b, pb = _scalar_ptr(scale_b, dev)
    keep_r, pr = (None, None) if scale_result is None else _scalar_ptr(scale_result, dev)
    with torch.cuda.device(dev):
        n = int(L.mmb200_workspace_bytes_split(c.M, c.N, c.K, c.decision.S))
        ws = torch.empty(n, dtype=torch.uint8, device=dev)
        rc = L.mmb200_quantize_scaled_mm_ws(xs.data_ptr(), xs.stride(0) if c.M > 1 else c.K,
                                            1 if xs.dtype == torch.float32 else 2, pq, xq.data_ptr(), c.K, bt.data_ptr(),
                                            ldb, _lib.FMT_CODES[c.fb], y.data_ptr(), c.N,
                                            _lib.OUT_CODES[OUT_DTYPE_NAMES[c.od]], c.M, c.N, c.K, c.preset.code,
                                            int(bool(use_fast_accum)), c.decision.S, _lib.SCHEME_CODES[c.scheme], pa, pb,
                                            pr, ws.data_ptr(), n, _stream_ptr(dev))
    _lib.check("mmb200_quantize_scaled_mm_ws", rc)
    del keep_q, keep_a, keep_b, keep_r, ws
    return (y, xq) if return_codes else y


def accumulate(a, b, *, use_fast_accum, profile=None, splitk="auto", backend="auto",
               out_dtype_for_split=torch.float32):
    """fp32 [M, N] accumulator of a [M, K] x b [N, K]^T before alpha, as the profile's cuBLAS computes it (the
    reference's mmaemu.accumulate, mmaemu/api.py:382-421). a, b: FP8 tensors of any K, alignment or layout.
    use_fast_accum has no default on purpose. The split decision is keyed with out_dtype_for_split."""
    for name, v in (("a", a), ("b", b)):
        if not isinstance(v, torch.Tensor):
            raise TypeError(f"accumulate(): argument '{name}' must be Tensor, not {type(v).__name__}")
    if not isinstance(use_fast_accum, bool) and type(use_fast_accum).__name__ != "bool_":
        raise TypeError(f"accumulate(): use_fast_accum must be bool, not {type(use_fast_accum).__name__}")
    if not isinstance(out_dtype_for_split, torch.dtype):
        raise TypeError("accumulate(): out_dtype_for_split must be a torch.dtype")
    fa, fb = fmt_of(a.dtype), fmt_of(b.dtype)
    if a.dim() != 2 or b.dim() != 2:
        raise ValueError(f"accumulate(): expected a [M, K] and b [N, K], got {tuple(a.shape)} and {tuple(b.shape)}")
    if a.shape[1] != b.shape[1]:
        raise ValueError(f"accumulate(): K mismatch: a is {tuple(a.shape)}, b is {tuple(b.shape)}")
    if a.device != b.device:
        raise ValueError(f"accumulate(): a and b are on different devices ({a.device}, {b.device})")
    if torch.is_grad_enabled() and (a.requires_grad or b.requires_grad):
        raise UnsupportedFeatureError("inference only: an input requires grad while grad mode is enabled")
    prof = get_profile(profile)
    preset = get_preset(prof.preset)
    _emit_maturity(prof, preset)
    M, K, N = a.shape[0], a.shape[1], b.shape[0]
    fast = bool(use_fast_accum)
    if M == 0 or N == 0 or K == 0:
        return torch.zeros(M, N, dtype=torch.float32, device=a.device)
    decision = resolve_splitk(M, N, K, a_dtype=a.dtype, b_dtype=b.dtype, out_dtype=out_dtype_for_split,
                              use_fast_accum=fast, profile=prof, splitk=splitk, layout_std=True)
    kernel = _kernel_choice(backend)
    _require_device(a.device)
    scheme = check_plan(preset, K, decision.S, decision.scheme, fast)
    dev = a.device
    au, bu = a.detach().contiguous(), b.detach().contiguous()
    acc = torch.empty((M, N), dtype=torch.float32, device=dev)
    L = _lib.load()
    with torch.cuda.device(dev):
        ws, ws_ptr, ws_bytes = _workspace(L, kernel, au.data_ptr(), K, bu.data_ptr(), K, M, N, K, preset.code,
                                          decision.S, dev)
        rc = L.mmb200_accumulate_ws(au.data_ptr(), K, _lib.FMT_CODES[fa], bu.data_ptr(), K, _lib.FMT_CODES[fb],
                                    acc.data_ptr(), N, M, N, K, preset.code, int(fast), decision.S,
                                    _lib.SCHEME_CODES[scheme], _kernel_code(kernel), ws_ptr, ws_bytes, _stream_ptr(dev))
    _lib.check("mmb200_accumulate_ws", rc)
    del ws
    return acc


def explain(input, mat2, scale_a, scale_b, bias=None, scale_result=None, out_dtype=None, use_fast_accum=False,
            *, out=None, profile=None, splitk="auto", backend="auto") -> CallPlan:
    """Validate a scaled_mm call and report what it would do, without computing (same arguments as scaled_mm)."""
    cp = CallPlan()
    try:
        with warnings.catch_warnings(record=True) as seen:
            warnings.simplefilter("always")
            c = _prepare(input, mat2, scale_a, scale_b, bias, scale_result, out_dtype, use_fast_accum, out, profile,
                         splitk, backend, dry=True)
            if not (c.early or c.unchanged_out):
                check_plan(c.preset, c.K, c.decision.S, c.decision.scheme, bool(use_fast_accum))
        cp.warnings = list(c.notes) + [str(w.message) for w in seen]
        cp.profile, cp.preset, cp.preset_maturity = c.profile.name, c.preset.name, c.preset.maturity
        cp.split = c.decision
        if c.early:
            cp.backend = "none (zero-size result)"
        elif c.unchanged_out:
            cp.backend = "none (out= is returned unchanged)"
        else:
            cp.backend = "cuda:b200" if c.kernel == "auto" else f"cuda:b200-{c.kernel}"
    except Exception as e:  # noqa: BLE001 - explain reports instead of raising
        cp.validation = (type(e).__name__, str(e))
        try:
            prof = get_profile(profile)
            preset = get_preset(prof.preset)
            cp.profile, cp.preset, cp.preset_maturity = prof.name, preset.name, preset.maturity
        except Exception:  # noqa: BLE001
            pass
    return cp


# torch.compile must not trace into these entry points (they call a foreign library through ctypes)
scaled_mm = torch.compiler.disable(scaled_mm)
accumulate = torch.compiler.disable(accumulate)
explain = torch.compiler.disable(explain)
