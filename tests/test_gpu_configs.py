"""The benchmark configurations beyond the headline one, at their own sizes, on a B200 (-m gpu).

Every case goes through the public call (mmaemu_b200.scaled_mm / sharded_scaled_mm) with the split-K decision taken
from the profile's table, and is compared bit for bit with the oracle on sampled rows and columns of the full result
(an output depends on its own row of A and column of B only, so a sampled sub-problem is the same computation).

  * tall-skinny mixed-format GEMMs (e5m2 x e4m3, K up to 32768) with fp32 and bf16 outputs, plus table rows that split;
  * the projection stack of a 7B-width and a 40B-width FP8 model under profile 'hopper-te', with amax-derived scales;
  * a row slab of the 32768 x 32768 x 8192 sharded GEMM with special codes injected, fp16 (overflow) and bf16 outputs.
"""
import warnings

import numpy as np
import pytest
import torch

import datagen
import mmaemu_b200 as mm
from mmaemu_b200.splitk import resolve_splitk
from oracle import oracle

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
F8 = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}
OUT = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}
VIEW = {4: (torch.int32, np.uint32), 2: (torch.int16, np.uint16)}


def bits(t):
    tv, nv = VIEW[t.element_size()]
    return t.detach().cpu().contiguous().view(tv).numpy().view(nv)


def quiet(fn, *a, **k):
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        return fn(*a, **k)


def check_sampled(y, a, b, rows, cols, label, **oracle_kw):
    got = bits(y[torch.as_tensor(rows, device=y.device)][:, torch.as_tensor(cols, device=y.device)])
    want = oracle.scaled_mm(a[rows], b[cols], **oracle_kw)
    bad = np.argwhere(got != want)
    assert bad.size == 0, f"{label}: {len(bad)} of {want.size} sampled outputs differ, first at {bad[0]}"


# ---------------------------------------------------------------------------------------------------------------
TALL = [(M, K, out) for M in (16, 64, 128) for K in (8192, 16384, 32768) for out in ("float32", "bfloat16")]


@pytest.mark.parametrize("M,K,out", TALL, ids=lambda v: str(v))
def test_tall_skinny_mixed_formats(M, K, out):
    """hopper, N = 4096, A e5m2 and B e4m3 from N(0, 1) * 8. The split comes from the H100 table; where the table and
    its envelope do not know the shape the call must raise SplitKUnknownError exactly as the reference does, and the
    numerics are then checked with explicit contiguous splits (the scheme the H100 table maps every split to)."""
    N = 4096
    rng = np.random.default_rng(M * 7 + K)
    a = datagen._round_to(rng.standard_normal((M, K)) * 8, "e5m2")
    b = datagen._round_to(rng.standard_normal((N, K)) * 8, "e4m3")
    ta, tb = torch.from_numpy(a).to(DEV).view(F8["e5m2"]), torch.from_numpy(b).to(DEV).view(F8["e4m3"])
    sa, sb = torch.tensor(2.0 ** -5, device=DEV), torch.tensor(2.0 ** -4, device=DEV)
    rows = np.arange(M) if M <= 16 else np.sort(rng.choice(M, 16, replace=False))
    cols = np.sort(rng.choice(N, 48, replace=False))
    for fast in (False, True):
        try:
            d = quiet(resolve_splitk, M, N, K, a_dtype="e5m2", b_dtype="e4m3", out_dtype=out, use_fast_accum=fast,
                      profile="hopper")
            splits = ["auto"]
            plan = (d.S, d.scheme)
        except mm.SplitKUnknownError:
            with pytest.raises(mm.SplitKUnknownError):
                quiet(mm.scaled_mm, ta, tb.t(), sa, sb, out_dtype=OUT[out], use_fast_accum=fast, profile="hopper")
            splits = [(2, "contiguous"), (5, "contiguous")]
            plan = None
        for sk in splits:
            S, scheme = plan if sk == "auto" else sk
            y = quiet(mm.scaled_mm, ta, tb.t(), sa, sb, out_dtype=OUT[out], use_fast_accum=fast, profile="hopper",
                      splitk=sk)
            assert y.shape == (M, N) and y.dtype == OUT[out]
            check_sampled(y, a, b, rows, cols, f"M={M} K={K} {out} fast={fast} split={S}/{scheme}", scale_a=2.0 ** -5,
                          scale_b=2.0 ** -4, out=out, fmt_a="e5m2", fmt_b="e4m3", preset="hopper", fast=fast, S=S,
                          scheme=scheme)


@pytest.mark.parametrize("profile,M,N,K", [("hopper-te", 16, 8192, 28672), ("hopper", 16, 3584, 18944)],
                         ids=("te-16x8192x28672", "torch-16x3584x18944"))
@pytest.mark.parametrize("out", ("float32", "bfloat16"))
def test_tall_skinny_table_rows_that_split(out, profile, M, N, K):
    """e5m2 x e4m3 rows of the H100 table whose recorded numSplitsK is above 1 (contiguous K ranges, the partial sums
    added in fp32 before the epilogue): one under Transformer Engine's 32 MiB workspace, one under torch's 1 MiB."""
    rng = np.random.default_rng(5)
    a = datagen._round_to(rng.standard_normal((M, K)) * 8, "e5m2")
    b = datagen._round_to(rng.standard_normal((N, K)) * 8, "e4m3")
    ta, tb = torch.from_numpy(a).to(DEV).view(F8["e5m2"]), torch.from_numpy(b).to(DEV).view(F8["e4m3"])
    sa, sb = torch.tensor(0.03125, device=DEV), torch.tensor(0.0625, device=DEV)
    cols = np.sort(rng.choice(N, 64, replace=False))
    for fast in (False, True):
        d = quiet(resolve_splitk, M, N, K, a_dtype="e5m2", b_dtype="e4m3", out_dtype=out, use_fast_accum=fast,
                  profile=profile)
        assert d.S > 1 and d.scheme == "contiguous" and d.source == "table", d
        y = quiet(mm.scaled_mm, ta, tb.t(), sa, sb, out_dtype=OUT[out], use_fast_accum=fast, profile=profile)
        check_sampled(y, a, b, np.arange(M), cols, f"{out} fast={fast}", scale_a=0.03125, scale_b=0.0625, out=out,
                      fmt_a="e5m2", fmt_b="e4m3", preset="hopper", fast=fast, S=d.S, scheme=d.scheme)


# ---------------------------------------------------------------------------------------------------------------
def quantise(x, fmt="e4m3"):
    """Per-tensor amax scaling as FP8 training recipes do it: scale = amax / max_finite; codes of x / scale."""
    amax = float(np.abs(x).max())
    scale = np.float32(amax / (448.0 if fmt == "e4m3" else 57344.0))
    return datagen._round_to(x / scale, fmt), scale


STACK = [("7B qkv", 8192, 5760, 1920), ("7B out", 8192, 1920, 1920), ("40B qkv", 8192, 24576, 8192)]


@pytest.mark.parametrize("name,M,N,K", STACK, ids=[s[0] for s in STACK])
def test_projection_stack_hopper_te(name, M, N, K):
    """hopper-te: activations N(0, 1), weights N(0, 0.02), both e4m3 with amax-derived scales, bf16 output."""
    rng = np.random.default_rng(K + N)
    a, sa = quantise(rng.standard_normal((M, K)).astype(np.float32))
    w, sw = quantise((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    ta, tw = torch.from_numpy(a).to(DEV).view(F8["e4m3"]), torch.from_numpy(w).to(DEV).view(F8["e4m3"])
    rows = np.sort(rng.choice(M, 24, replace=False))
    cols = np.sort(rng.choice(N, 40, replace=False))
    for fast in (True, False):                         # Transformer Engine's forward GEMMs use fast accumulation
        d = quiet(resolve_splitk, M, N, K, a_dtype="e4m3", b_dtype="e4m3", out_dtype="bfloat16", use_fast_accum=fast,
                  profile="hopper-te")
        y = quiet(mm.scaled_mm, ta, tw.t(), torch.tensor(sa, device=DEV), torch.tensor(sw, device=DEV),
                  out_dtype=torch.bfloat16, use_fast_accum=fast, profile="hopper-te")
        check_sampled(y, a, w, rows, cols, f"{name} fast={fast}", scale_a=sa, scale_b=sw, out="bfloat16",
                      preset="hopper", fast=fast, S=d.S, scheme=d.scheme)


# ---------------------------------------------------------------------------------------------------------------
def with_specials(rng, rows, K, nan_rows):
    """N(0, 1) * 16 in e4m3 with 1 % of the positions replaced by subnormals and +-max-finite codes, and the NaN codes
    0x7F / 0xFF at one seeded position of each row in `nan_rows` (a NaN poisons its whole output row or column, so
    they are kept to a few rows to leave finite outputs to compare)."""
    x = datagen._round_to(rng.standard_normal((rows, K)) * 16, "e4m3")
    mask = rng.random((rows, K)) < 0.01
    pool = np.array([0x01, 0x03, 0x07, 0x81, 0x86, 0x7E, 0xFE], np.uint8)
    x[mask] = pool[rng.integers(0, len(pool), int(mask.sum()))]
    for i, r in enumerate(nan_rows):
        x[r, rng.integers(0, K)] = 0x7F if i % 2 == 0 else 0xFF
    return x


@pytest.mark.parametrize("profile", ("hopper", "ada"))
@pytest.mark.parametrize("out", ("float16", "bfloat16"))
def test_sharded_slab_with_specials(profile, out):
    """One rank's share of the 32768 x 32768 x 8192 GEMM on 16 GPUs' worth of rows (2048 of them; every other slab is
    the same computation on other rows), all 32768 columns, through sharded_scaled_mm. The split decision is the one
    of the full shape. fp16 outputs overflow to infinity for the largest sums."""
    from mmaemu_b200.sharding import sharded_scaled_mm
    Mfull, Mloc, N, K = 32768, 2048, 32768, 8192
    rng = np.random.default_rng(11 if profile == "hopper" else 12)
    nan_r = rng.choice(Mloc, 8, replace=False)
    nan_c = rng.choice(N, 32, replace=False)
    a = with_specials(rng, Mloc, K, nan_r)
    b = with_specials(rng, N, K, nan_c)
    ta, tb = torch.from_numpy(a).to(DEV).view(F8["e4m3"]), torch.from_numpy(b).to(DEV).view(F8["e4m3"])
    sa, sb = torch.tensor(1.0, device=DEV), torch.tensor(1.25, device=DEV)   # sums of about 3e4: some exceed fp16's range
    d = quiet(resolve_splitk, Mfull, N, K, a_dtype="e4m3", b_dtype="e4m3", out_dtype=out, use_fast_accum=False,
              profile=profile)
    assert d.S == 1
    y = quiet(mm.scaled_mm, ta, tb.t(), sa, sb, out_dtype=OUT[out], profile=profile, splitk=1)
    y2 = quiet(sharded_scaled_mm, ta, tb.t(), sa, sb, out_dtype=OUT[out], profile=profile, splitk=1,
               input_is_local=True, full_rows=Mloc)                                 # one process: the slab is the whole call
    assert torch.equal(y.view(torch.int16), y2.view(torch.int16))
    rows = np.concatenate([nan_r[:3], rng.choice(Mloc, 21, replace=False)])
    cols = np.concatenate([nan_c[:4], rng.choice(N, 44, replace=False)])
    check_sampled(y, a, b, rows, cols, f"{profile} {out}", scale_a=1.0, scale_b=1.25, out=out, preset=profile,
                  fast=False)
    got = bits(y)
    exp_mask, nan_bits = (0x7C00, 0x7FFF) if out == "float16" else (0x7F80, 0x7FFF)
    assert (got[nan_r] == nan_bits).all() and (got[:, nan_c] == nan_bits).all()      # canonical NaN rows and columns
    finite_part = np.delete(np.delete(got, nan_r, axis=0), nan_c, axis=1)
    inf = ((finite_part & 0x7FFF) == exp_mask)
    assert not ((finite_part & 0x7FFF) > exp_mask).any()                             # no NaN anywhere else
    if out == "float16":
        assert inf.any()                                                             # sums beyond 65504 become +-inf
    else:
        assert not inf.any()
