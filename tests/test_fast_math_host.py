"""The arithmetic of the fast CUDA kernel, compiled for the host and checked against the oracle's block model.

mmaemu_b200/csrc/fast_math.cuh holds the kernel's scalar steps (byte-parallel decode, packed exponent pass, offset
accumulator with round-toward-zero FMA, floor/truncation fix, deferred cut) as host+device functions. This test builds
them with g++ (directed rounding through the floating-point environment) and compares whole chains, bit for bit, with
oracle.dot on adversarial data classes, for every format pair and both presets. No GPU involved."""
import ctypes
import subprocess
from pathlib import Path

import numpy as np
import pytest

import datagen
from oracle import oracle

HERE = Path(__file__).resolve().parent
SRC = HERE / "host" / "fast_math_host.cpp"
LIB = HERE / "host" / "_build" / "libfast_math_host.so"
FMT = {"e4m3": 0, "e5m2": 1, "e4m3-pow": 4, "e5m2-pow": 5}     # "-pow": block exponents from sums of powers (tensor-core pass)


@pytest.fixture(scope="module")
def lib():
    hdr = HERE.parent / "mmaemu_b200" / "csrc" / "fast_math.cuh"
    if not LIB.exists() or LIB.stat().st_mtime < max(SRC.stat().st_mtime, hdr.stat().st_mtime):
        LIB.parent.mkdir(exist_ok=True)
        subprocess.run(["g++", "-O1", "-frounding-math", "-fPIC", "-shared", "-std=c++17", "-x", "c++", str(SRC), "-o",
                        str(LIB)], check=True)
    L = ctypes.CDLL(str(LIB))
    L.fast_math_chains.argtypes = [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 6 + [ctypes.c_void_p]
    L.fast_math_chains.restype = ctypes.c_int
    L.fast_math_power_sum_check.restype = ctypes.c_int
    L.fast_math_power5_check.restype = ctypes.c_int
    return L


def chains(L, a, b, fa, fb, nfma, chain_len=0):
    out = np.zeros(a.shape[0], np.float32)
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    assert L.fast_math_chains(a.ctypes.data, b.ctypes.data, a.shape[0], a.shape[1], FMT[fa], FMT[fb], nfma, chain_len,
                              out.ctypes.data) == 0
    return out.view(np.uint32)


@pytest.mark.parametrize("nfma", (16, 32))
@pytest.mark.parametrize("fmts", (("e4m3", "e4m3"), ("e5m2", "e4m3"), ("e4m3", "e5m2"), ("e5m2", "e5m2")), ids="x".join)
@pytest.mark.parametrize("cls", datagen.CLASSES)
def test_chains_equal_the_block_model(lib, cls, fmts, nfma):
    rng = np.random.default_rng(len(cls) * 131 + nfma)
    for K in (16, 48, 256, 1936):
        a = datagen.codes(rng, 96, K, fmts[0], cls, 0)
        b = datagen.codes(rng, 96, K, fmts[1], cls, 1)
        got = chains(lib, a, b, fmts[0], fmts[1], nfma)
        want = oracle.dot(a, b, None, fmt_a=fmts[0], fmt_b=fmts[1], preset=nfma)
        bad = np.nonzero(got != want)[0]
        assert bad.size == 0, f"{cls} K={K}: {bad.size} of {got.size} chains differ; row {bad[0]}: " \
                              f"{got[bad[0]]:#x} != {want[bad[0]]:#x}"


@pytest.mark.parametrize("nfma", (16, 32))
@pytest.mark.parametrize("cls", datagen.CLASSES)
def test_power_sum_exponent_pass_equals_the_block_model(lib, cls, nfma):
    rng = np.random.default_rng(len(cls) * 17 + nfma)
    for K in (16, 48, 256, 1936, 8192):
        a = datagen.codes(rng, 64, K, "e4m3", cls, 0)
        b = datagen.codes(rng, 64, K, "e4m3", cls, 1)
        want = oracle.dot(a, b, None, preset=nfma)
        assert np.array_equal(chains(lib, a, b, "e4m3-pow", "e4m3-pow", nfma), want), (cls, K)
        if K >= 256:
            slow = np.array([oracle.accumulate(a[i:i + 1], b[i:i + 1], preset=nfma, fast=False)[0, 0] for i in range(8)])
            got = chains(lib, a[:8], b[:8], "e4m3-pow", "e4m3-pow", nfma, chain_len=128)
            assert np.array_equal(got, slow), (cls, K)


@pytest.mark.parametrize("nfma", (16, 32))
@pytest.mark.parametrize("fmts", (("e5m2", "e4m3"), ("e4m3", "e5m2")), ids="x".join)
@pytest.mark.parametrize("cls", datagen.CLASSES)
def test_power_sum_exponent_pass_of_the_mixed_pairs(lib, cls, fmts, nfma):
    """Mixed pairs: powers of 32 and the larger of the 16-term sums (block_exponent_pow5_raw), summed in two different
    orders and rounding modes by the host harness."""
    assert lib.fast_math_power5_check() == 0
    rng = np.random.default_rng(len(cls) * 29 + nfma)
    for K in (16, 48, 256, 1936, 8192):
        a = datagen.codes(rng, 64, K, fmts[0], cls, 0)
        b = datagen.codes(rng, 64, K, fmts[1], cls, 1)
        want = oracle.dot(a, b, None, fmt_a=fmts[0], fmt_b=fmts[1], preset=nfma)
        got = chains(lib, a, b, fmts[0] + "-pow", fmts[1] + "-pow", nfma)
        assert np.array_equal(got, want), (cls, K)
        if K >= 256:
            slow = np.array([oracle.accumulate(a[i:i + 1], b[i:i + 1], fmt_a=fmts[0], fmt_b=fmts[1], preset=nfma,
                                               fast=False)[0, 0] for i in range(8)])
            got = chains(lib, a[:8], b[:8], fmts[0] + "-pow", fmts[1] + "-pow", nfma, chain_len=128)
            assert np.array_equal(got, slow), (cls, K)


def test_long_chains_with_growing_accumulators(lib):
    rng = np.random.default_rng(3)
    a = datagen.codes(rng, 24, 32768, "e5m2", "gauss40")
    b = np.abs(datagen.codes(rng, 24, 32768, "e4m3", "max_mag").view(np.int8)).view(np.uint8)   # one-signed: sums grow
    a &= 0x7F
    for nfma in (16, 32):
        assert np.array_equal(chains(lib, a, b, "e5m2", "e4m3", nfma),
                              oracle.dot(a, b, None, fmt_a="e5m2", fmt_b="e4m3", preset=nfma))


def test_slow_accumulation_chunks(lib):
    rng = np.random.default_rng(4)
    for K in (128, 400, 1024):
        a = datagen.codes(rng, 40, K, "e4m3", "gauss40")
        b = datagen.codes(rng, 40, K, "e4m3", "block_exponents")
        for nfma in (16, 32):
            got = chains(lib, a, b, "e4m3", "e4m3", nfma, chain_len=128)
            want = np.array([oracle.accumulate(a[i:i + 1], b[i:i + 1], preset=nfma, fast=False)[0, 0] for i in range(40)])
            assert np.array_equal(got, want)


def test_nonfinite_codes_count_as_zero(lib):
    rng = np.random.default_rng(5)
    a = rng.integers(0, 256, (64, 64), dtype=np.uint8)
    b = rng.integers(0, 256, (64, 64), dtype=np.uint8)
    for fa, fb in (("e4m3", "e5m2"), ("e5m2", "e4m3")):
        clean = [np.where((x & 0x7F) == 0x7F, 0, x) if f == "e4m3" else np.where((x & 0x7C) == 0x7C, 0, x)
                 for x, f in ((a, fa), (b, fb))]
        want = oracle.dot(clean[0].astype(np.uint8), clean[1].astype(np.uint8), None, fmt_a=fa, fmt_b=fb, preset=32)
        assert np.array_equal(chains(lib, a, b, fa, fb, 32), want)


def test_tensor_core_exponent_pass_decode(lib):
    """The exponent field read off a sum of powers 64^(ea + eb) is the block exponent for every sum a tensor core can
    return, and the per-code powers are 2^(6 ea)."""
    assert lib.fast_math_power_sum_check() == 0


def test_quantise_prologue_equals_torch(lib):
    """quantise_e4m3 against torch's clamp + conversion on the CPU: every fp32 value with a 12-bit mantissa prefix across
    the whole exponent range (all rounding ties of the E4M3 grid among them), random values, zeros, infinities, NaN."""
    import torch
    rng = np.random.default_rng(3)
    hi = (np.arange(1 << 21, dtype=np.uint32) << 11)                     # sign, exponent, 12 mantissa bits
    spots = np.array([0x00000000, 0x80000000, 0x7F800000, 0xFF800000, 0x7FC00000, 0xFFC00000, 0x43E00000, 0x43E80000,
                      0x43F00000, 0x3A800000, 0x3A000000, 0x39800000, 0x3A400000, 0x3AC00000], dtype=np.uint32)
    rnd = rng.integers(0, 1 << 32, 1 << 20, dtype=np.uint64).astype(np.uint32)
    near = (rng.standard_normal(1 << 20) * 64).astype(np.float32).view(np.uint32)
    bits = np.concatenate([hi, spots, rnd, near])
    v = bits.view(np.float32)
    out = np.zeros(v.size, np.uint8)
    lib.fast_math_quantise_e4m3.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    lib.fast_math_quantise_e4m3(v.ctypes.data, v.size, out.ctypes.data)
    want = torch.from_numpy(v.copy()).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    bad = np.nonzero(out != want)[0]
    assert bad.size == 0, f"{bad.size} differ; first {bits[bad[0]]:#010x}: {out[bad[0]]:#x} != {want[bad[0]]:#x}"
