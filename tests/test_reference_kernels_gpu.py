"""The reference's own CUDA kernels, loaded by the reference's stock loader on the same B200, against this package:
full outputs, bit for bit (-m gpu).

The unmodified reference package is expected under baseline/_ref/ (baseline/install_reference.py puts it there; it is
never committed). `mmaemu.scaled_mm(..., backend="cuda:h4" | "cuda:h1" | "cuda:v4" | "cuda:v1")` goes through the
reference's registry, fatbin loader and smoke gate (astding/mmaemu mmaemu/backends/registry.py:194-267,
mmaemu/backends/cuda/modules.py:192-226); the same arguments then go to mmaemu_b200.scaled_mm. The kernels of the
reference serve E4M3 x E4M3 only, so the format pair is fixed; everything else varies: both presets, fast and slow
accumulation, explicit splits, every output dtype, the reference's smoke and conformance data classes, the headline
4096-cube and the projection-stack shapes.

If a reference kernel cannot be loaded on this device the case is skipped with the reference's own reason.
"""
import sys
import warnings
import zlib
from pathlib import Path

import numpy as np
import pytest
import torch

import datagen

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT / "baseline"))
import install_reference  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
E4M3 = torch.float8_e4m3fn
KERNELS = {"h4": "hopper", "h1": "hopper", "v4": "ada", "v1": "ada"}
VIEW = {4: torch.int32, 2: torch.int16, 1: torch.uint8}


@pytest.fixture(scope="module")
def ref():
    if not install_reference.add_to_path():
        pytest.skip("the reference package is not installed under baseline/_ref (python baseline/install_reference.py)")
    import mmaemu
    return mmaemu


@pytest.fixture(scope="module")
def available(ref):
    """{kernel: None or the reference's reason for not offering it on this device}"""
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        st = ref.backends_status(DEV)
    out = {}
    for k in KERNELS:
        s = st.get(f"cuda:{k}")
        out[k] = None if (s is not None and s.available) else (s.reason if s is not None else "not discovered")
        print(f"reference cuda:{k} on {torch.cuda.get_device_name(DEV)}: "
              f"{'available (' + str(s.source) + ')' if out[k] is None else out[k]}")
    return out


def need(available, kernel):
    if available[kernel] is not None:
        pytest.skip(f"reference backend cuda:{kernel} unavailable here: {available[kernel]}")


def bits(t):
    return t.detach().contiguous().view(VIEW[t.element_size()])


def both(ref, kernel, a_u8, b_u8, sa, sb, **kw):
    """(reference kernel's result, this package's result) of the same scaled_mm call, as integer bit tensors."""
    import mmaemu_b200 as mm
    a = torch.as_tensor(a_u8).to(DEV).view(E4M3)
    bt = torch.as_tensor(b_u8).to(DEV).view(E4M3)
    s1, s2 = torch.tensor(sa, dtype=torch.float32, device=DEV), torch.tensor(sb, dtype=torch.float32, device=DEV)
    profile = KERNELS[kernel]
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        want = ref.scaled_mm(a, bt.t(), s1, s2, profile=profile, backend=f"cuda:{kernel}", **kw)
        got = mm.scaled_mm(a, bt.t(), s1, s2, profile=profile, backend="cuda:b200", **kw)
    torch.cuda.synchronize(DEV)
    assert got.shape == want.shape and got.dtype == want.dtype
    return bits(want), bits(got)


def assert_same(want, got, label):
    bad = int((want != got).sum())
    assert bad == 0, f"{label}: {bad} of {want.numel()} outputs differ from the reference kernel"


@pytest.mark.parametrize("kernel", list(KERNELS))
def test_smoke_data_of_the_reference(ref, available, kernel):
    """The two cases of the reference's own smoke gate (gaussian x 40, adversarial row groups), as accumulate()."""
    need(available, kernel)
    import mmaemu_b200 as mm
    from mmaemu.backends.cuda import selftest
    for a, b, _ in selftest._smoke_cases(KERNELS[kernel]):
        a, b = a.to(DEV).view(E4M3), b.to(DEV).view(E4M3)
        for fast in (True, False):
            with warnings.catch_warnings():
                warnings.simplefilter("ignore")
                want = ref.accumulate(a, b, use_fast_accum=fast, profile=KERNELS[kernel], splitk=1,
                                      backend=f"cuda:{kernel}")
                got = mm.accumulate(a, b, use_fast_accum=fast, profile=KERNELS[kernel], splitk=1)
            assert_same(bits(want), bits(got), f"{kernel} smoke {tuple(a.shape)} fast={fast}")


CONF = [(cls, M, N, K) for cls in datagen.CLASSES for (M, N, K) in ((65, 63, 48), (129, 257, 1920), (200, 127, 1920))]


@pytest.mark.parametrize("kernel", list(KERNELS))
@pytest.mark.parametrize("cls,M,N,K", CONF, ids=lambda v: str(v))
def test_conformance_classes(ref, available, kernel, cls, M, N, K):
    """The data classes of the reference's kernel conformance tests on ragged shapes (tests/test_kernels_ieee.py:34-36
    uses M in {1, 65, 129, 200}, N in {1, 63, 127, 257}, K in {16, 48, 1920}); K and N are multiples of 16 here because
    the call goes through scaled_mm's own checks."""
    need(available, kernel)
    N16 = -(-N // 16) * 16
    rng = np.random.default_rng(zlib.crc32(f"{cls}-{M}-{N}-{K}".encode()))
    a = datagen.codes(rng, M, K, "e4m3", cls, side=0)
    b = datagen.codes(rng, N16, K, "e4m3", cls, side=1)
    for fast, out in ((True, torch.float32), (False, torch.bfloat16)):
        want, got = both(ref, kernel, a, b, 0.75, 1.5, out_dtype=out, use_fast_accum=fast, splitk=1)
        assert_same(want, got, f"{kernel} {cls} {M}x{N16}x{K} fast={fast}")


SPLITS = {"hopper": [(2, "contiguous"), (5, "contiguous"), (24, "contiguous")],
          "ada": [(2, "serial"), (3, "pairwise"), (12, "serial"), (29, "pairwise")]}


@pytest.mark.parametrize("kernel", list(KERNELS))
def test_explicit_splits_and_output_dtypes(ref, available, kernel):
    need(available, kernel)
    rng = np.random.default_rng(11)
    M, N, K = 136, 208, 6144
    a = datagen.codes(rng, M, K, "e4m3", "gauss40")
    b = datagen.codes(rng, N, K, "e4m3", "all_codes")
    outs = (torch.float32, torch.bfloat16, torch.float16, torch.float8_e4m3fn)
    for i, sk in enumerate(SPLITS[KERNELS[kernel]]):
        for fast in (True, False):
            out = outs[(i + int(fast)) % len(outs)]
            want, got = both(ref, kernel, a, b, 2.0 ** -9, 0.5, out_dtype=out, use_fast_accum=fast, splitk=sk)
            assert_same(want, got, f"{kernel} split {sk} fast={fast} {out}")


def test_nan_codes_and_fp16_overflow(ref, available):
    """Rows and columns with NaN codes, saturated codes and scales that overflow fp16: the non-finite patch and the
    output conversion after the reference's kernel (h1 propagates NaN itself; h4 relies on the plan's patch)."""
    rng = np.random.default_rng(5)
    M, N, K = 256, 256, 2048
    a = datagen.codes(rng, M, K, "e4m3", "max_mag")
    b = datagen.codes(rng, N, K, "e4m3", "max_mag", side=1)
    a[7, 100], a[200, 0], b[31, 2047], b[32, 5] = 0x7F, 0xFF, 0x7F, 0xFF
    for kernel in KERNELS:
        if available[kernel] is not None:
            continue
        want, got = both(ref, kernel, a, b, 1.0, 0.25, out_dtype=torch.float16, use_fast_accum=True, splitk=1)
        assert_same(want, got, f"{kernel} NaN codes, fp16 overflow")
        assert int((want == 0x7FFF).sum()) >= M + N - 4 and int(((want & 0x7FFF) == 0x7C00).sum()) > 0


@pytest.mark.parametrize("kernel,fast", [("h4", False), ("h4", True), ("v4", True), ("h1", True)])
def test_headline_cube(ref, available, kernel, fast):
    """The headline workload, 4096 x 4096 x 4096 with N(0, 1) * 4 operands and bf16 output, full output."""
    need(available, kernel)
    g = torch.Generator().manual_seed(2)
    a = (torch.randn(4096, 4096, generator=g) * 4).clamp(-448, 448).to(E4M3).view(torch.uint8)
    b = (torch.randn(4096, 4096, generator=g) * 4).clamp(-448, 448).to(E4M3).view(torch.uint8)
    want, got = both(ref, kernel, a, b, 0.3, 2.5, out_dtype=torch.bfloat16, use_fast_accum=fast, splitk=1)
    assert_same(want, got, f"{kernel} 4096 cube fast={fast}")


@pytest.mark.parametrize("N,K", [(5760, 1920), (1920, 1920)])
def test_projection_stack_shapes(ref, available, N, K):
    """8192 tokens through the fused-QKV and output projections of a 7B-width FP8 model (amax-derived scales,
    use_fast_accum=True as Transformer Engine sets it), h4 against this package, full output."""
    need(available, "h4")
    g = torch.Generator().manual_seed(40)
    x = torch.randn(8192, K, generator=g)
    w = torch.randn(N, K, generator=g) * 0.02
    sx, sw = 448.0 / float(x.abs().max()), 448.0 / float(w.abs().max())
    a = (x * sx).clamp(-448, 448).to(E4M3).view(torch.uint8)
    b = (w * sw).clamp(-448, 448).to(E4M3).view(torch.uint8)
    want, got = both(ref, "h4", a, b, 1.0 / sx, 1.0 / sw, out_dtype=torch.bfloat16, use_fast_accum=True, splitk=1)
    assert_same(want, got, f"h4 8192x{N}x{K}")
