"""Replay of the two H100 PCIe hardware recordings of astding/mmaemu (docs/validation_logs/2026-10-15/h100-probe and
2026-10-16/h100-splitk-sweep, results/live_jobs.tar.gz: 4,194 live torch._scaled_mm calls), as the reference's
tools/replay_h100_log.py does it: every call is recomputed with the logged cuBLASLt split passed explicitly and the
sha256 of the full output is compared with the H100's; the split the profile resolves on its own must equal the logged
one wherever it resolves; the calls the H100 rejected must be rejected.

Without a GPU: the fixture, the input generators, the split decisions and rejections of all calls, and the oracle
against the hardware on the small calls. On a B200 (-m gpu): all calls through mmaemu_b200.scaled_mm.
"""
import dataclasses
import gzip
import hashlib
import json
import warnings
from functools import lru_cache

import numpy as np
import pytest
import torch

import golden_cases as G
import h100_inputs
import mmaemu_b200 as mm
from mmaemu_b200.platforms import get_profile
from mmaemu_b200.splitk import resolve_splitk
from oracle import oracle

F8 = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}
CHUNK = 96


@lru_cache(maxsize=None)
def jobs():
    return json.loads(gzip.open(G.GOLDEN / "h100_live.json.gz").read())["jobs"]


def profile_for(ws: int):
    """The hopper platform with the call's logged workspace (torch's 1 MiB is 'hopper' itself, 0 is 'hopper-ws0')."""
    base = get_profile("hopper")
    if ws == 0:
        return get_profile("hopper-ws0")
    if ws == base.workspace_bytes:
        return base
    return dataclasses.replace(base, name=f"hopper-ws{ws}", workspace_bytes=ws)


def test_fixture():
    js = jobs()
    assert len(js) == 4194 and sum(1 for j in js if j.get("rejected")) == 27
    assert len({j["id"] for j in js}) == len(js)
    assert {j["src"].split("/")[0] for j in js} == {"probe", "sweep"}
    assert sum(1 for j in js if j.get("S", 1) > 1) == 3465 and max(j.get("S", 1) for j in js) == 24
    assert all(len(j["sha256"]) == 64 for j in js if not j.get("rejected"))


def test_torch_generator_equals_the_numpy_one():
    js = jobs()
    picked = [js[i] for i in range(0, len(js), 97)] + [j for j in js if j["data"]["kind"] == "adv"][:4]
    for j in picked:
        small = dict(j, M=min(j["M"], 70), N=min(j["N"], 33))
        a, b = h100_inputs.make_inputs(small)
        a2, b2 = h100_inputs.make_inputs_torch(small, chunk_elements=1 << 16)
        assert np.array_equal(a, a2.numpy()) and np.array_equal(b, b2.numpy()), j["id"]


def test_split_decisions_and_rejections_of_every_call():
    """splitk='auto' on the call's platform: a decision (table or envelope) must be the logged one; shapes off the
    table's grid may be unknown. The H100's rejections are exactly the profile's reject rule."""
    agree = unknown = m6 = 0
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        for j in jobs():
            p = profile_for(j["ws"])
            rule = p.rejection(j["fa"], j["fb"], j["out"])
            assert (rule is not None) == bool(j.get("rejected")), j["id"]
            if j.get("rejected"):
                continue
            try:
                d = resolve_splitk(j["M"], j["N"], j["K"], a_dtype=j["fa"], b_dtype=j["fb"], out_dtype=j["out"],
                                   use_fast_accum=bool(j["fast"]), profile=p)
            except mm.SplitKUnknownError:
                unknown += 1
                continue
            assert (d.S, d.scheme) == (j["S"], j["scheme"]), (j["id"], d)
            agree += 1
            m6 += j["src"] == "probe/m6_live"
    # the reference's own replays of the two recordings report 1,341 + 248 agreeing decisions and no disagreement; all
    # 1,000 calls of the heuristics part (m6) must resolve
    assert agree + unknown == 4167 and agree >= 1341 + 248 and m6 == 1000


def small_calls(limit_gmac=0.012, count=160):
    js = [j for j in jobs() if not j.get("rejected") and j["M"] * j["N"] * j["K"] <= limit_gmac * 1e9]
    step = max(1, len(js) // count)
    return js[::step][:count]


@pytest.mark.parametrize("j", small_calls(), ids=lambda j: j["id"])
def test_oracle_equals_the_hardware_on_small_calls(j):
    a, b = h100_inputs.make_inputs(j)
    y = oracle.scaled_mm(a, b, j["scale_a"], j["scale_b"], out=j["out"], fmt_a=j["fa"], fmt_b=j["fb"], preset="hopper",
                         fast=bool(j["fast"]), S=j["S"], scheme=j["scheme"], scale_result=j["scale_result"])
    assert hashlib.sha256(np.ascontiguousarray(y).tobytes()).hexdigest() == j["sha256"]


def chunks():
    js = sorted(jobs(), key=lambda j: (j["M"] + j["N"]) * j["K"])
    return [js[i:i + CHUNK] for i in range(0, len(js), CHUNK)]


@pytest.mark.gpu
@pytest.mark.parametrize("chunk", chunks(), ids=lambda c: f"{c[0]['id']}..{c[-1]['id']}")
def test_replay_on_gpu(chunk):
    dev = torch.device("cuda:0")
    views = {4: torch.int32, 2: torch.int16, 1: torch.uint8}
    bad = []
    for j in chunk:
        a8, b8 = h100_inputs.make_inputs_torch(j, device=dev)
        a, b = a8.view(F8[j["fa"]]), b8.view(F8[j["fb"]])
        sa = torch.tensor(j["scale_a"], dtype=torch.float32, device=dev)
        sb = torch.tensor(j["scale_b"], dtype=torch.float32, device=dev)
        sr = None if j["scale_result"] is None else torch.tensor(j["scale_result"], dtype=torch.float32, device=dev)
        kw = dict(scale_result=sr, out_dtype=getattr(torch, j["out"]), use_fast_accum=bool(j["fast"]),
                  profile=profile_for(j["ws"]))
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            if j.get("rejected"):
                with pytest.raises(mm.ReferenceRejectsError):
                    mm.scaled_mm(a, b.t(), sa, sb, splitk=1, **kw)
                continue
            y = mm.scaled_mm(a, b.t(), sa, sb, splitk=1 if j["S"] == 1 else (j["S"], j["scheme"]), **kw)
        raw = y.contiguous().view(views[y.element_size()]).cpu().numpy().tobytes()
        if hashlib.sha256(raw).hexdigest() != j["sha256"]:
            bad.append(j["id"])
    assert not bad, f"{len(bad)} of {len(chunk)} calls differ from the H100: {bad[:8]}"
