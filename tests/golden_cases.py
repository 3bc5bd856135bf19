"""Uniform access to the golden fixtures of tests/golden (see tests/golden/make_golden.py for what each file holds).

Every fixture is turned into `Case` records: operand codes, plan parameters, scales and the expected output, either as
bits (`want`) or as the sha256 of the bits (`want_sha256`, the H100 live calls). `evaluate(case, run)` runs a case
through any implementation with the signature of oracle.scaled_mm / oracle.accumulate and returns the mismatch count.
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass
from functools import lru_cache
from pathlib import Path

import numpy as np

GOLDEN = Path(__file__).resolve().parent / "golden"
LATE_PROFILE = "b200-mma-sync-experimental"
# preset number of each profile at the C boundary and in the oracle (products per block; + 256: late accumulator)
NFMA = {"ada": 16, "ada-te": 16, "ada-ws0": 16, "hopper": 32, "hopper-te": 32, "hopper-ws0": 32, LATE_PROFILE: 288}


@dataclass
class Case:
    id: str
    load: object                 # () -> (a [M, K] uint8, b [N, K] uint8)
    fa: str
    fb: str
    profile: str
    fast: bool
    S: int
    scheme: str
    out: str
    scale_a: np.float32
    scale_b: np.float32
    scale_result: object         # np.float32 or None
    api: str = "scaled_mm"       # or "accumulate" (fp32 accumulator before alpha)
    want: object = None          # () -> ndarray of bits
    want_sha256: str | None = None
    gmac: float = 0.0

    @property
    def nfma(self) -> int:
        return NFMA[self.profile]


def _f32(bits):
    return None if bits is None else np.array([bits], dtype=np.uint32).view(np.float32)[0]


@lru_cache(maxsize=None)
def _npz(name):
    return np.load(GOLDEN / name, allow_pickle=False)


def reference_cases(late: bool = False):
    """The reference's outputs on seeded inputs: the early-accumulator presets (default), or the cases of the
    late-accumulator preset that the same file holds (late=True)."""
    idx = json.loads((GOLDEN / "reference_cases.json").read_text())["cases"]
    out = []
    for i, c in enumerate(idx):
        if (c["profile"] == LATE_PROFILE) != late:
            continue
        z = lambda i=i: _npz("reference_cases.npz")  # noqa: E731
        out.append(Case(id=f"ref{i:02d}-{c['profile']}-{c['fa']}x{c['fb']}-{c['out']}-{'fast' if c['fast'] else 'slow'}"
                           f"-S{c['S']}{c['scheme'] if c['S'] > 1 else ''}{'-special' if c['special'] else ''}",
                        load=lambda z=z, i=i: (z()[f"a{i}"], z()[f"b{i}"]), fa=c["fa"], fb=c["fb"],
                        profile=c["profile"], fast=c["fast"], S=c["S"], scheme=c["scheme"], out=c["out"],
                        scale_a=_f32(c["scale_a_bits"]), scale_b=_f32(c["scale_b_bits"]),
                        scale_result=_f32(c["scale_result_bits"]), api=c["api"],
                        want=lambda z=z, i=i: z()[f"y{i}"], gmac=c["M"] * c["N"] * c["K"] / 1e9))
    return out


def late_preset_cases():
    return reference_cases(late=True)


def epilogue_tie_cases():
    idx = json.loads((GOLDEN / "hw_epilogue_ties.json").read_text())
    out = []
    for i, c in enumerate(idx["cases"]):
        z = lambda: _npz("hw_epilogue_ties.npz")  # noqa: E731
        out.append(Case(id=f"tie{i:02d}-{c['kind']}-{c['out']}-{'fast' if c['fast'] else 'slow'}",
                        load=lambda z=z, i=i: (z()[f"a{i}"], z()["b"]), fa="e4m3", fb="e4m3", profile="ada",
                        fast=c["fast"], S=1, scheme="none", out=c["out"], scale_a=_f32(c["scale_a_bits"]),
                        scale_b=_f32(c["scale_b_bits"]), scale_result=None,
                        want=lambda z=z, i=i: z()[f"y{i}"], gmac=4 * 768 * 1920 / 1e9))
    return out


def epilogue_extract_cases():
    idx = json.loads((GOLDEN / "hw_epilogue_extract.json").read_text())
    out = []
    for ci, c in enumerate(idx["cases"]):
        for oi, o in enumerate(c["outputs"]):
            z = lambda: _npz("hw_epilogue_extract.npz")  # noqa: E731
            out.append(Case(id=f"hwx{ci}_{oi:02d}-{c['fa']}x{c['fb']}-{o['out']}-S{o['S']}",
                            load=lambda z=z, ci=ci: (z()[f"a{ci}"], z()[f"b{ci}"]), fa=c["fa"], fb=c["fb"],
                            profile="ada", fast=o["fast"], S=o["S"], scheme=o["scheme"], out=o["out"],
                            scale_a=_f32(o["scale_a_bits"]), scale_b=_f32(o["scale_b_bits"]),
                            scale_result=_f32(o["scale_result_bits"]),
                            want=lambda z=z, ci=ci, oi=oi: z()[f"y{ci}_{oi}"]))
    return out


def h100_cases(max_gmac: float | None = None):
    """The H100 PCIe live calls that computed (the two calls the H100 rejected are in h100_rejected())."""
    import h100_inputs
    jobs = json.loads((GOLDEN / "h100_mini.json").read_text())["jobs"]
    out = []
    for j in jobs:
        if "error" in j["expect"]:
            continue
        g = j["M"] * j["N"] * j["K"] / 1e9
        if max_gmac is not None and g > max_gmac:
            continue
        out.append(Case(id=f"h100-{j['id']}-{j['fa']}x{j['fb']}-{j['out']}-S{j['S']}",
                        load=lambda j=j: h100_inputs.make_inputs(j), fa=j["fa"], fb=j["fb"],
                        profile="hopper-ws0" if j["ws"] == 0 else "hopper", fast=bool(j["fast"]), S=j["S"],
                        scheme=j["scheme"] if j["S"] > 1 else "none", out=j["out"],
                        scale_a=np.float32(j["scale_a"]), scale_b=np.float32(j["scale_b"]),
                        scale_result=None if j["scale_result"] is None else np.float32(j["scale_result"]),
                        want_sha256=j["expect"]["sha256"], gmac=g))
    return out


def h100_rejected():
    jobs = json.loads((GOLDEN / "h100_mini.json").read_text())["jobs"]
    return [j for j in jobs if "error" in j["expect"]]


def evaluate(case: Case, scaled_mm, accumulate) -> str | None:
    """Run `case` through (scaled_mm, accumulate) callables that take the oracle's keyword arguments and return bit
    arrays. Returns None when the output matches, else a one-line description of the mismatch."""
    a, b = case.load()
    kw = dict(fmt_a=case.fa, fmt_b=case.fb, preset=case.nfma, fast=case.fast, S=case.S, scheme=case.scheme)
    if case.api == "accumulate":
        got = accumulate(a, b, **kw)
    else:
        got = scaled_mm(a, b, case.scale_a, case.scale_b, out=case.out, scale_result=case.scale_result, **kw)
    got = np.ascontiguousarray(got)
    if case.want_sha256 is not None:
        h = hashlib.sha256(got.tobytes()).hexdigest()
        return None if h == case.want_sha256 else f"{case.id}: sha256 {h} != recorded {case.want_sha256}"
    want = case.want()
    if got.shape != want.shape or got.dtype != want.dtype:
        return f"{case.id}: got {got.dtype}{got.shape}, want {want.dtype}{want.shape}"
    bad = got != want
    if not bad.any():
        return None
    i = tuple(int(x) for x in np.argwhere(bad)[0])
    return f"{case.id}: {int(bad.sum())} of {want.size} outputs differ; first at {i}: got {got[i]:#x}, want {want[i]:#x}"
