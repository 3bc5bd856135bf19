"""Parity of the CUDA path with the oracle and the golden fixtures, through the C ABI. Needs a B200 (-m gpu).

What is covered, in the order the reference's own kernel tests cover it (tests/test_kernels_ieee.py,
tests/test_h100_mini.py, tests/test_epilogue.py of astding/mmaemu):
  - the golden fixtures: reference outputs, RTX 4060 hardware bits, H100 PCIe sha256 (all 122 calls);
  - a conformance matrix: 8 data classes x ragged M / N x K {16, 48, 1920} x both presets x three format pairs;
  - every accumulation plan: slow accumulation, serial / pairwise S in {2, 3, 8, 12, 29}, contiguous S in {2..8, 24},
    ragged K, empty splits;
  - non-finite inputs, every output dtype, leading dimensions larger than K, any byte value never faults;
  - size-independent properties at full benchmark sizes (row / column independence, sign symmetry).
Every comparison is bit for bit."""
import zlib

import numpy as np
import pytest

import datagen
import golden_cases as G
from oracle import oracle

pytestmark = pytest.mark.gpu
KERNELS = ("integer", "auto", "staged", "staged-whole", "staged-rows")     # "staged*": with scratch memory (tests/gpu_runner.py)


@pytest.fixture(scope="module")
def gpu():
    import gpu_runner
    return gpu_runner


def _same(got, want, label):
    bad = got != want
    if bad.any():
        i = tuple(int(x) for x in np.argwhere(bad)[0])
        pytest.fail(f"{label}: {int(bad.sum())} of {want.size} outputs differ; first at {i}: got {got[i]:#x}, "
                    f"want {want[i]:#x}")


# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("case", G.reference_cases() + G.late_preset_cases() + G.epilogue_tie_cases()
                         + G.epilogue_extract_cases(), ids=lambda c: c.id)
def test_golden(gpu, case, kernel):
    msg = G.evaluate(case, *gpu.for_kernel(kernel))
    assert msg is None, msg


@pytest.mark.parametrize("case", G.h100_cases(), ids=lambda c: c.id)
def test_h100_live_calls(gpu, case):
    msg = G.evaluate(case, *gpu.for_kernel("auto"))
    assert msg is None, msg


# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("preset", (16, 32))
@pytest.mark.parametrize("fmts", (("e4m3", "e4m3"), ("e5m2", "e4m3"), ("e4m3", "e5m2")), ids="x".join)
@pytest.mark.parametrize("cls", datagen.CLASSES)
def test_conformance_matrix(gpu, cls, fmts, preset, kernel):
    rng = np.random.default_rng(zlib.crc32(repr((cls, fmts, preset)).encode()))
    for M, N in ((1, 1), (65, 63), (129, 127), (200, 257)):
        for K in (16, 48, 1920):
            a = datagen.codes(rng, M, K, fmts[0], cls, 0)
            b = datagen.codes(rng, N, K, fmts[1], cls, 1)
            want = oracle.accumulate(a, b, fmt_a=fmts[0], fmt_b=fmts[1], preset=preset, fast=True)
            _same(gpu.chain(a, b, fmt_a=fmts[0], fmt_b=fmts[1], preset=preset, kernel=kernel), want,
                  f"{cls} {M}x{N}x{K}")


@pytest.mark.parametrize("fmts", (("e4m3", "e4m3"), ("e5m2", "e4m3"), ("e4m3", "e5m2"), ("e5m2", "e5m2")), ids="x".join)
@pytest.mark.parametrize("cls", datagen.CLASSES)
def test_late_accumulator_preset(gpu, cls, fmts):
    """b200_mma_sync (preset number 288: 32 products aligned on the largest product exponent with 25 fraction bits,
    block sums cut to 24 bits and added to the accumulator in fp32) on the integer kernel, chains and whole calls
    with non-finite codes, against the oracle; plans the reference does not characterise are refused."""
    rng = np.random.default_rng(zlib.crc32(repr((cls, fmts, 288)).encode()))
    for M, N in ((1, 1), (65, 63), (200, 257)):
        for K in (16, 40, 1920):
            a = datagen.codes(rng, M, K, fmts[0], cls, 0)
            b = datagen.codes(rng, N, K, fmts[1], cls, 1)
            want = oracle.accumulate(a, b, fmt_a=fmts[0], fmt_b=fmts[1], preset=288, fast=True)
            for kernel in ("auto", "staged"):
                _same(gpu.accumulate(a, b, fmt_a=fmts[0], fmt_b=fmts[1], preset=288, fast=True, kernel=kernel), want,
                      f"{cls} {M}x{N}x{K} {kernel}")
    a, b = datagen.codes(rng, 70, 512, fmts[0], cls, 0), datagen.codes(rng, 90, 512, fmts[1], cls, 1)
    a[3, 100], b[5, 7] = 0x7F, (0x7F if fmts[1] == "e4m3" else 0x7C)                 # NaN row, NaN / +Inf column
    for out in ("float16", "float8_e4m3fn"):
        want = oracle.scaled_mm(a, b, 0.5, 3.0, out=out, fmt_a=fmts[0], fmt_b=fmts[1], preset=288, fast=True)
        _same(gpu.scaled_mm(a, b, 0.5, 3.0, out=out, fmt_a=fmts[0], fmt_b=fmts[1], preset=288, fast=True), want, out)
    for kw in (dict(fast=False), dict(fast=True, S=2, scheme="contiguous"), dict(fast=True, kernel="fast")):
        with pytest.raises(RuntimeError, match="UNSUPPORTED|unsupported|not supported"):
            gpu.accumulate(a, b, fmt_a=fmts[0], fmt_b=fmts[1], preset=288, **kw)


@pytest.mark.parametrize("preset", (16, 32))
@pytest.mark.parametrize("fmts", (("e4m3", "e4m3"), ("e5m2", "e4m3"), ("e4m3", "e5m2")), ids="x".join)
@pytest.mark.parametrize("cls", datagen.CLASSES)
def test_packed_integer_exponent_pass_for_tensor_core_pairs(gpu, cls, preset, fmts):
    """Every pair but E5M2 x E5M2 takes its exponent pass from the tensor cores by default (powers of 256 for
    E4M3 x E4M3, powers of 32 and the larger of two 16-term sums for the mixed pairs); the packed-integer pass serves
    them too (MMAEMU_B200_TC_EPASS=0) and must give the same bits: chains, a slow-accumulation plan and a split
    plan, on the 8-row-slot kernels and on the 16-row kernels."""
    rng = np.random.default_rng(zlib.crc32(repr((cls, preset, fmts, "int")).encode()))
    f = dict(fmt_a=fmts[0], fmt_b=fmts[1])
    for M, N, K in ((65, 63, 48), (200, 257, 1920), (9, 140, 1056)):
        a = datagen.codes(rng, M, K, fmts[0], cls, 0)
        b = datagen.codes(rng, N, K, fmts[1], cls, 1)
        _same(gpu.chain(a, b, preset=preset, kernel="staged-int", **f), oracle.accumulate(a, b, preset=preset, fast=True, **f),
              f"{cls} {M}x{N}x{K}")
        sch = "contiguous" if preset == 32 else "pairwise"
        for kw in (dict(fast=False, S=1, scheme="none"), dict(fast=True, S=3, scheme=sch)):
            _same(gpu.accumulate(a, b, preset=preset, kernel="staged-int", **kw, **f),
                  oracle.accumulate(a, b, preset=preset, **kw, **f), f"{cls} {M}x{N}x{K} {kw}")


PLANS = ([(16, False, 1, "none"), (32, False, 1, "none")]
         + [(16, f, S, sch) for sch in ("serial", "pairwise") for S in (2, 3, 8, 12, 29) for f in (True, False)]
         + [(32, f, S, "contiguous") for S in (2, 3, 4, 5, 6, 7, 8, 24) for f in (True, False)]
         + [(32, True, 3, "pairwise"), (16, False, 4, "contiguous")])      # custom-preset combinations


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("plan", PLANS, ids=lambda p: f"nfma{p[0]}-{'fast' if p[1] else 'slow'}-S{p[2]}-{p[3]}")
def test_plans(gpu, plan, kernel):
    preset, fast, S, scheme = plan
    rng = np.random.default_rng(S * 7 + preset)
    for M, N, K in ((33, 70, 64), (17, 48, 528), (40, 40, 2048), (5, 130, 1936)):
        a = datagen.codes(rng, M, K, "e4m3", "gauss40")
        b = datagen.codes(rng, N, K, "e4m3", "block_exponents")
        kw = dict(preset=preset, fast=fast, S=S, scheme=scheme)
        _same(gpu.accumulate(a, b, kernel=kernel, **kw), oracle.accumulate(a, b, **kw), f"{M}x{N}x{K}")


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("out", ("float32", "bfloat16", "float16", "float8_e4m3fn", "float8_e5m2"))
@pytest.mark.parametrize("fmts", (("e4m3", "e4m3"), ("e5m2", "e4m3"), ("e4m3", "e5m2"), ("e5m2", "e5m2")), ids="x".join)
def test_nonfinite_inputs_and_output_dtypes(gpu, fmts, out, kernel):
    rng = np.random.default_rng(11)
    M, N, K = 70, 90, 256
    for scale in (1e-3, 0.37, 300.0):
        a = datagen.codes(rng, M, K, fmts[0], "gauss40")
        b = datagen.codes(rng, N, K, fmts[1], "all_codes")
        for x, fmt in ((a, fmts[0]), (b, fmts[1])):
            nan, inf = (0x7F, None) if fmt == "e4m3" else (0x7E, 0x7C)
            for _ in range(3):
                x[rng.integers(0, x.shape[0]), rng.integers(0, K)] = nan | (rng.integers(0, 2) << 7)
                if inf is not None:
                    x[rng.integers(0, x.shape[0]), rng.integers(0, K)] = inf | (rng.integers(0, 2) << 7)
        kw = dict(out=out, fmt_a=fmts[0], fmt_b=fmts[1], preset=32, fast=True,
                  scale_result=0.6 if out.startswith("float8") else None)
        _same(gpu.scaled_mm(a, b, scale, 1.7, kernel=kernel, **kw), oracle.scaled_mm(a, b, scale, 1.7, **kw), out)


@pytest.mark.parametrize("kernel", ("auto", "staged", "staged-whole", "staged-rows"))
@pytest.mark.parametrize("fmts", (("e4m3", "e4m3"), ("e5m2", "e4m3"), ("e4m3", "e5m2"), ("e5m2", "e5m2")), ids="x".join)
def test_at_most_16_rows(gpu, fmts, kernel):
    """Calls with at most 16 rows run on kernels of their own (both operands decoded in the kernel, all warps on the 16
    rows, K slices for plans with several chains): every row count's edge, ragged column counts, padded leading
    dimensions, non-finite codes in both operands -- also where only one K slice sees them -- every output dtype,
    slow and fast accumulation, a split plan."""
    rng = np.random.default_rng(zlib.crc32(repr(fmts).encode()))
    outs = ("float32", "bfloat16", "float16", "float8_e4m3fn", "float8_e5m2")
    n = 0
    for M in (1, 7, 16):
        for N, K in ((40, 48), (300, 2048), (128, 4096)):
            a = datagen.codes(rng, M, K, fmts[0], "gauss40")
            b = datagen.codes(rng, N, K, fmts[1], "all_codes")
            nan_a, nan_b = (0x7F if fmts[0] == "e4m3" else 0x7E), (0x7F if fmts[1] == "e4m3" else 0x7C)   # NaN; NaN or +Inf
            a[M - 1, K - 3] = nan_a                                   # seen by the last K slice only
            b[N // 2, 5] = nan_b | 0x80                               # seen by the first one only
            if fmts[0] == "e5m2" and M > 1:
                a[0, K // 2] = 0x7C                                   # +Inf: the IEEE class needs the walk over K
            for fast, S, scheme in ((False, 1, "none"), (True, 1, "none"), (True, 3, "contiguous")):
                out = outs[n % 5]
                n += 1
                kw = dict(out=out, fmt_a=fmts[0], fmt_b=fmts[1], preset=32, fast=fast, S=S, scheme=scheme,
                          scale_result=1.5 if out.startswith("float8") else None)
                _same(gpu.scaled_mm(a, b, 0.02, 0.7, kernel=kernel, ld_pad=16 * (n % 2), **kw),
                      oracle.scaled_mm(a, b, 0.02, 0.7, **kw), f"{M}x{N}x{K} {out} fast={fast} S={S}")


@pytest.mark.parametrize("kernel", KERNELS)
def test_every_byte_value_and_padded_leading_dimensions(gpu, kernel):
    rng = np.random.default_rng(5)
    for fmts in (("e4m3", "e4m3"), ("e5m2", "e4m3")):
        a = rng.integers(0, 256, (96, 320), dtype=np.uint8)
        b = rng.integers(0, 256, (80, 320), dtype=np.uint8)
        kw = dict(out="bfloat16", fmt_a=fmts[0], fmt_b=fmts[1], preset=16, fast=False)
        _same(gpu.scaled_mm(a, b, 0.5, 0.25, kernel=kernel, ld_pad=48, **kw), oracle.scaled_mm(a, b, 0.5, 0.25, **kw),
              "any byte")


def test_empty_and_degenerate_shapes(gpu):
    a = np.zeros((0, 64), np.uint8)
    b = np.zeros((5, 64), np.uint8)
    assert gpu.accumulate(a, b).shape == (0, 5)
    assert gpu.accumulate(b, a).shape == (5, 0)
    z = gpu.accumulate(np.zeros((3, 0), np.uint8), np.zeros((4, 0), np.uint8))
    assert z.shape == (3, 4) and not z.any()
    one = np.full((1, 16), 0x38, np.uint8)                       # 1.0
    assert gpu.chain(one, one, preset=16)[0, 0] == np.float32(16).view(np.uint32)


# ---------------------------------------------------------------------------------------------------------------
def test_full_size_properties(gpu):
    """At the benchmark's size (4096^3, far beyond what the CPU oracle checks in seconds): sampled rows and columns of
    the full output equal the oracle on the corresponding sub-problem (outputs depend only on their own row and column),
    and negating A negates every finite nonzero output (truncation toward zero is sign symmetric)."""
    rng = np.random.default_rng(2)
    M = N = K = 4096
    a = datagen._round_to(rng.standard_normal((M, K)) * 4, "e4m3")
    b = datagen._round_to(rng.standard_normal((N, K)) * 4, "e4m3")
    full = gpu.accumulate(a, b, preset=32, fast=True)
    rows = rng.choice(M, 24, replace=False)
    cols = rng.choice(N, 40, replace=False)
    _same(full[np.ix_(rows, cols)], oracle.accumulate(a[rows], b[cols], preset=32, fast=True), "sampled block")
    neg = gpu.accumulate(a ^ 0x80, b, preset=32, fast=True)
    nz = (full & 0x7FFFFFFF) != 0
    assert np.array_equal(neg[nz], full[nz] ^ 0x80000000) and not (neg[~nz] & 0x7FFFFFFF).any()


def test_host_entry_point(gpu):
    """mmb200_scaled_mm_host: host operands in, host result out."""
    import ctypes
    from mmaemu_b200 import _lib
    rng = np.random.default_rng(9)
    M, N, K = 130, 96, 528
    a = datagen.codes(rng, M, K, "e5m2", "gauss40")
    b = datagen.codes(rng, N, K, "e4m3", "gauss40")
    d = np.zeros((M, N), np.uint16)
    sr = None
    rc = _lib.load().mmb200_scaled_mm_host(a.ctypes.data, K, 1, b.ctypes.data, K, 0, d.ctypes.data, N, 2, M, N, K, 32, 0,
                                           3, 3, ctypes.c_float(0.011), ctypes.c_float(2.5), sr, 0, None)
    _lib.check("mmb200_scaled_mm_host", rc)
    want = oracle.scaled_mm(a, b, 0.011, 2.5, out="float16", fmt_a="e5m2", fmt_b="e4m3", preset=32, fast=False, S=3,
                            scheme="contiguous")
    _same(d, want, "host entry point")
