"""Split-K resolution on the host: decisions the emulated platforms are known to take, the order of the resolution
steps, warnings, and -- when a checkout of the reference is present -- agreement with the reference's resolver on
seeded random queries (decision, source, verified flag, error and warning classes)."""
import os
import random
import sys
import warnings
from pathlib import Path

import pytest
import torch

import mmaemu_b200 as mm
from mmaemu_b200 import splitk as sk

E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2
BF16, F32 = torch.bfloat16, torch.float32


def resolve(M, N, K, a=E4, b=E4, out=BF16, fast=True, **kw):
    return sk.resolve_splitk(M, N, K, a_dtype=a, b_dtype=b, out_dtype=out, use_fast_accum=fast, **kw)


def test_explicit_forms():
    d = resolve(64, 64, 4096, profile="ada", splitk=1)
    assert (d.S, d.scheme, d.source, d.verified) == (1, "none", "explicit", True)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        assert resolve(64, 64, 4096, profile="ada", splitk=(3, "pairwise")).splitk == sk.SplitK(3, "pairwise")
        assert resolve(64, 64, 4096, profile="hopper", splitk=sk.SplitK(4, "contiguous")).S == 4
    with pytest.raises(ValueError):
        resolve(64, 64, 4096, profile="ada", splitk=2)
    with pytest.raises(TypeError):
        resolve(64, 64, 4096, profile="ada", splitk="two")
    with pytest.raises(ValueError):
        sk.SplitK(1, "serial")
    with pytest.raises(ValueError):
        sk.SplitK(2, "none")


def test_workspace0_never_splits():
    for p in ("ada-ws0", "hopper-ws0"):
        d = resolve(16, 64, 16384, profile=p)
        assert (d.S, d.source) == (1, "workspace0")


def test_table_rows_and_envelopes():
    assert resolve(256, 256, 256, profile="ada", fast=False).source == "table"            # benchmark config 1
    d = resolve(4096, 4096, 4096, profile="hopper")                                       # benchmark config 2
    assert (d.S, d.source) == (1, "table")
    for K, N in ((1920, 5760), (1920, 1920), (8192, 24576)):                              # Evo-2-like projections
        d = resolve(8192, N, K, profile="hopper-te")
        assert (d.S, d.source) == (1, "table")
    d = resolve(32768, 32768, 8192, profile="hopper")                                     # sharded config: envelope
    assert (d.S, d.source, d.verified) == (1, "envelope", True)
    with pytest.warns(mm.UnvalidatedEnvelopeWarning):
        d = resolve(32768, 32768, 8192, profile="hopper-te", dry=True)
    assert (d.S, d.source, d.verified) == (1, "envelope", False)
    assert resolve(32768, 32768, 8192, profile="ada").source == "envelope"
    with pytest.raises(mm.SplitKUnknownError):
        resolve(256, 256, 256, profile="hopper")                                          # K below the envelope range
    with pytest.raises(mm.SplitKUnknownError):
        resolve(32768, 32768, 8192, profile="hopper", strict=True)
    with pytest.raises(mm.SplitKUnknownError):
        resolve(64, 64, 4096, profile="hopper-experimental")


def test_recorded_splits_of_the_h100():
    import json
    import golden_cases as G
    jobs = json.loads((G.GOLDEN / "h100_mini.json").read_text())["jobs"]
    hits = 0
    for j in jobs:
        if j["src"] != "m6_live" or j["ws"] != 1 << 20 or "error" in j["expect"]:
            continue
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            d = sk.resolve_splitk(j["M"], j["N"], j["K"], a_dtype=j["fa"], b_dtype=j["fb"],
                                  out_dtype=getattr(torch, j["out"]), use_fast_accum=bool(j["fast"]), profile="hopper")
        assert (d.S, d.scheme) == (j["S"], j["scheme"] if j["S"] > 1 else "none"), j["id"]
        hits += d.S > 1
    assert hits >= 10


def test_unverified_combination_warns_once():
    sk._reset_warnings_for_tests()
    with pytest.warns(mm.UnverifiedSplitWarning):
        resolve(64, 64, 4096, profile="hopper", splitk=(2, "serial"))
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        resolve(64, 64, 4096, profile="hopper", splitk=(2, "serial"))                     # second time: silent
    with pytest.warns(mm.UnverifiedSplitWarning):
        resolve(64, 64, 4096, profile="hopper", splitk=(2, "serial"), dry=True)           # dry: every time


REFERENCE = os.environ.get("MMAEMU_REFERENCE", str(Path(__file__).resolve().parents[2] / "reference"))


@pytest.mark.skipif(not os.path.isfile(os.path.join(REFERENCE, "mmaemu", "platform", "splitk_table.py")),
                    reason="no checkout of the reference")
def test_agrees_with_the_reference_resolver():
    sys.path.insert(0, REFERENCE)
    sys.dont_write_bytecode = True
    from mmaemu.platform.splitk_table import resolve_splitk as ref
    rnd = random.Random(7)
    dims = [1, 16, 32, 48, 64, 96, 128, 192, 256, 512, 768, 1024, 1920, 2048, 4096, 5760, 8192, 12288, 16384, 32768]

    def run(fn, M, N, K, kw):
        with warnings.catch_warnings(record=True) as w:
            warnings.simplefilter("always")
            try:
                d = fn(M, N, K, **kw)
                return ("ok", d.S, d.scheme, d.source, d.verified, tuple(sorted(type(x.message).__name__ for x in w)))
            except Exception as e:  # noqa: BLE001
                return ("err", type(e).__name__)
    for _ in range(1500):
        M, N, K = rnd.choice(dims), rnd.choice(dims), rnd.choice(dims[1:])
        a, b = rnd.choice([(E4, E4), (E4, E5), (E5, E4)])
        kw = dict(a_dtype=a, b_dtype=b, out_dtype=rnd.choice([F32, BF16, torch.float16, E4, E5]),
                  use_fast_accum=rnd.random() < 0.5, dry=True, strict=rnd.random() < 0.2,
                  profile=rnd.choice(["ada", "ada-te", "ada-ws0", "hopper", "hopper-te", "hopper-ws0"]))
        assert run(sk.resolve_splitk, M, N, K, kw) == run(ref, M, N, K, kw), (M, N, K, kw)
