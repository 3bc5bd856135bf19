"""The Python entry points on a B200 (-m gpu): mmaemu_b200.scaled_mm / accumulate / the Backend object, bit for bit
against the oracle, plus the behaviours the reference pins at this boundary (tests/test_api.py and
tests/test_cuda_runtime.py of astding/mmaemu): out= handling, zero sizes, storage offsets, the current stream."""
import ctypes
import os
import warnings

import numpy as np
import pytest
import torch

import datagen
import mmaemu_b200 as mm
from mmaemu_b200 import _lib
from oracle import oracle

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
F8 = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}
NPV = {4: (torch.int32, np.uint32), 2: (torch.int16, np.uint16), 1: (torch.uint8, np.uint8)}


def bits(t):
    tv, nv = NPV[t.element_size()]
    return t.detach().cpu().contiguous().view(tv).numpy().view(nv)


def operands(M, N, K, fa="e4m3", fb="e4m3", seed=0, scale=4.0):
    rng = np.random.default_rng(seed)
    a = datagen._round_to(rng.standard_normal((M, K)) * scale, fa)
    b = datagen._round_to(rng.standard_normal((N, K)) * scale, fb)
    return a, b, torch.from_numpy(a).to(DEV).view(F8[fa]), torch.from_numpy(b).to(DEV).view(F8[fb])


@pytest.mark.parametrize("profile", ("hopper", "hopper-te", "hopper-ws0", "ada", "ada-te", "ada-ws0"))
@pytest.mark.parametrize("fast", (True, False))
def test_scaled_mm_profiles(profile, fast):
    a, b, ta, tb = operands(64, 128, 1024, seed=1)
    sa, sb = torch.tensor(0.5, device=DEV), torch.tensor(1.25, device=DEV)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        y = mm.scaled_mm(ta, tb.t(), sa, sb, out_dtype=torch.bfloat16, use_fast_accum=fast, profile=profile, splitk=1)
    want = oracle.scaled_mm(a, b, 0.5, 1.25, out="bfloat16", preset=profile.split("-")[0], fast=fast)
    assert y.dtype == torch.bfloat16 and y.device == DEV and np.array_equal(bits(y), want)


def test_late_accumulator_profile():
    """profile 'b200-mma-sync-experimental' (preset b200_mma_sync, mmaemu/platform/profiles.py:202-208): the reference's
    own outputs of the golden fixture through scaled_mm / accumulate, the maturity warning, and the reference's errors
    for what it does not characterise (slow accumulation, split-K, an automatic split decision)."""
    import golden_cases as G
    from mmaemu_b200 import numerics
    numerics._reset_warnings_for_tests()
    prof = G.LATE_PROFILE
    for i, c in enumerate(G.late_preset_cases()):
        a, b = c.load()
        ta, tb = torch.from_numpy(a).to(DEV).view(F8[c.fa]), torch.from_numpy(b).to(DEV).view(F8[c.fb])
        with warnings.catch_warnings(record=True) as seen:
            warnings.simplefilter("always")
            if c.api == "accumulate":
                y = mm.accumulate(ta, tb, use_fast_accum=True, profile=prof, splitk=1)
            else:
                sr = None if c.scale_result is None else torch.tensor(float(c.scale_result), device=DEV)
                y = mm.scaled_mm(ta, tb.t(), torch.tensor(float(c.scale_a), device=DEV),
                                 torch.tensor(float(c.scale_b), device=DEV), scale_result=sr,
                                 out_dtype=getattr(torch, c.out), use_fast_accum=True, profile=prof, splitk=1)
        assert np.array_equal(bits(y), c.want()), c.id
        experimental = [w for w in seen if issubclass(w.category, mm.ExperimentalPresetWarning)]
        assert len(experimental) == (1 if i == 0 else 0)                      # once per process and preset
        if i == 0:
            assert "NOT B200 cuBLAS" in str(experimental[0].message)
    a, b, ta, tb = operands(32, 48, 256, seed=9)
    s = torch.tensor(1.0, device=DEV)
    with pytest.raises(mm.UnsupportedFeatureError, match="slow accumulation"):
        mm.scaled_mm(ta, tb.t(), s, s, out_dtype=torch.bfloat16, use_fast_accum=False, profile=prof, splitk=1)
    with pytest.raises(mm.UnsupportedFeatureError, match="split-K"):
        mm.scaled_mm(ta, tb.t(), s, s, out_dtype=torch.bfloat16, use_fast_accum=True, profile=prof,
                     splitk=(2, "contiguous"))
    with pytest.raises(mm.SplitKUnknownError):
        mm.scaled_mm(ta, tb.t(), s, s, out_dtype=torch.bfloat16, use_fast_accum=True, profile=prof)
    with pytest.raises(mm.UnsupportedFeatureError):
        mm.quantized_scaled_mm(torch.randn(32, 256, device=DEV), s, tb.t(), s, s, out_dtype=torch.bfloat16,
                               use_fast_accum=True, profile=prof, splitk=1)
    # the chain function of the backend object (what the reference's executor calls) serves the preset as well
    from mmaemu_b200.backend import B200Backend

    class Req:
        device, fmt_a, fmt_b, preset = DEV, "e4m3", "e4m3", "b200_mma_sync"
    got = B200Backend().chain_fn(Req())(ta.view(torch.uint8), tb.view(torch.uint8))
    assert np.array_equal(bits(got), oracle.accumulate(a, b, preset=288, fast=True))
    assert "integer kernel only" in B200Backend("fast").supports(Req())


def test_config1_ada_256_cube():
    """M = N = K = 256, profile 'ada', seeds 0 / 1, scales 0.5 and 1.25, bf16 out, split-K from the table."""
    A = (torch.randn(256, 256, generator=torch.Generator().manual_seed(0)) * 2).to(torch.float8_e4m3fn)
    Bt = torch.randn(256, 256, generator=torch.Generator().manual_seed(1)).to(torch.float8_e4m3fn)
    for fast in (False, True):
        y = mm.scaled_mm(A.to(DEV), Bt.to(DEV).t(), torch.tensor(0.5, device=DEV), torch.tensor(1.25, device=DEV),
                         out_dtype=torch.bfloat16, use_fast_accum=fast, profile="ada")
        want = oracle.scaled_mm(A.view(torch.uint8).numpy(), Bt.view(torch.uint8).numpy(), 0.5, 1.25, out="bfloat16",
                                preset="ada", fast=fast)
        assert np.array_equal(bits(y), want)
    with pytest.raises(mm.SplitKUnknownError):
        mm.scaled_mm(A.to(DEV), Bt.to(DEV).t(), torch.tensor(0.5, device=DEV), torch.tensor(1.25, device=DEV),
                     out_dtype=torch.bfloat16, profile="hopper")


def _h100_jobs():
    import json
    import golden_cases as G
    return [j for j in json.loads((G.GOLDEN / "h100_mini.json").read_text())["jobs"]]


@pytest.mark.parametrize("j", _h100_jobs(), ids=lambda j: j["id"])
def test_h100_live_calls_through_scaled_mm(j):
    """The recorded H100 PCIe calls through the public entry point: the logged split passed explicitly must give the
    H100's output bits (sha256), the two calls the H100 rejected must raise, and splitk='auto' must resolve to the
    logged split wherever the profile's table holds the shape."""
    import hashlib
    import h100_inputs
    a, b = h100_inputs.make_inputs(j)
    ta = torch.from_numpy(a).to(DEV).view(F8[j["fa"]])
    tb = torch.from_numpy(b).to(DEV).view(F8[j["fb"]])
    sa, sb = torch.tensor(j["scale_a"], device=DEV), torch.tensor(j["scale_b"], device=DEV)
    sr = None if j["scale_result"] is None else torch.tensor(j["scale_result"], device=DEV)
    profile = {0: "hopper-ws0", 1 << 20: "hopper", 32 << 20: "hopper-te"}.get(j["ws"])
    kw = dict(scale_result=sr, out_dtype=getattr(torch, j["out"]), use_fast_accum=bool(j["fast"]),
              profile=profile or "hopper")
    if "error" in j["expect"]:
        with pytest.raises(getattr(mm, j["expect"]["error"])) as ei:
            mm.scaled_mm(ta, tb.t(), sa, sb, splitk=1, **kw)
        assert type(ei.value) is getattr(mm, j["expect"]["error"])
        return
    split = 1 if j["S"] == 1 else (j["S"], j["scheme"])
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        y = mm.scaled_mm(ta, tb.t(), sa, sb, splitk=split, **kw)
        cp = mm.explain(ta, tb.t(), sa, sb, splitk="auto", **kw)
    assert hashlib.sha256(bits(y).tobytes()).hexdigest() == j["expect"]["sha256"]
    if profile is not None and (j["src"] == "m6_live" or cp.validation == "ok"):
        assert cp.validation == "ok", cp.validation
        assert (cp.split.S, cp.split.scheme) == (j["S"], j["scheme"] if j["S"] > 1 else "none")


def test_out_argument_zero_sizes_and_offsets():
    a, b, ta, tb = operands(32, 48, 256, seed=4)
    s = torch.tensor(1.0, device=DEV)
    kw = dict(out_dtype=torch.float32, profile="ada", splitk=1)
    y = mm.scaled_mm(ta, tb.t(), s, s, **kw)
    out = torch.full((32, 48), 7.0, device=DEV)
    assert mm.scaled_mm(ta, tb.t(), s, s, out=out, **kw) is out and torch.equal(out, y)
    colmajor = torch.full((48, 32), 7.0, device=DEV).t()
    mm.scaled_mm(ta, tb.t(), s, s, out=colmajor, **kw)
    assert torch.equal(colmajor, y)
    with pytest.warns(UserWarning, match="resized"):
        wrong = torch.zeros(3, 5, device=DEV)
        mm.scaled_mm(ta, tb.t(), s, s, out=wrong, **kw)
    assert torch.equal(wrong, y)
    strided = torch.full((32, 96), 7.0, device=DEV)[:, ::2]
    with pytest.warns(UserWarning, match="unchanged"):
        r = mm.scaled_mm(ta, tb.t(), s, s, out=strided, **kw)
    assert r is strided and bool((strided == 7.0).all())
    z = mm.scaled_mm(ta[:, :0], tb[:, :0].t(), s, s, **kw)
    assert z.shape == (32, 48) and not bool(z.any())
    assert mm.scaled_mm(ta[:0], tb.t(), s, s, **kw).shape == (0, 48)
    # operands that are views into larger buffers (16-byte aligned offsets, padded leading dimension)
    big = torch.zeros(32 * 272 + 64, dtype=torch.uint8, device=DEV)
    va = big[32:32 + 32 * 272].view(32, 272)[:, :256]
    va.copy_(ta.view(torch.uint8))
    y2 = mm.scaled_mm(va.view(torch.float8_e4m3fn), tb.t(), s, s, **kw)
    assert torch.equal(y2, y)
    with pytest.raises(mm.ReferenceRejectsError):
        mm.scaled_mm(big[8:8 + 32 * 256].view(32, 256).view(torch.float8_e4m3fn), tb.t(), s, s, **kw)


def test_runs_on_the_current_stream():
    a, b, ta, tb = operands(256, 256, 2048, seed=5)
    s = torch.tensor(1.0, device=DEV)
    st = torch.cuda.Stream(DEV)
    with torch.cuda.stream(st):
        y = mm.scaled_mm(ta, tb.t(), s, s, out_dtype=torch.float32, profile="ada", splitk=1, use_fast_accum=True)
    st.synchronize()
    assert np.array_equal(bits(y), oracle.accumulate(a, b, preset="ada", fast=True))


def test_accumulate_any_k():
    for K in (8, 24, 200):
        a, b, ta, tb = operands(20, 31, K, "e4m3", "e5m2", seed=K)
        acc = mm.accumulate(ta, tb, use_fast_accum=False, profile="ada", splitk=1)
        assert np.array_equal(bits(acc), oracle.accumulate(a, b, fmt_a="e4m3", fmt_b="e5m2", preset="ada", fast=False))


def test_backend_object_chain_fn():
    from types import SimpleNamespace
    from mmaemu_b200.backend import BACKEND
    req = SimpleNamespace(device=DEV, fmt_a="e5m2", fmt_b="e4m3", preset="hopper")
    assert BACKEND.supports(req) is None
    fn = BACKEND.chain_fn(req)
    a, b, ta, tb = operands(65, 63, 48, "e5m2", "e4m3", seed=6)
    got = fn(ta.view(torch.uint8)[1:], tb)                      # a view with a storage offset
    assert np.array_equal(bits(got), oracle.accumulate(a[1:], b, fmt_a="e5m2", fmt_b="e4m3", preset="hopper", fast=True))
    with pytest.raises(ValueError):
        fn(ta.view(torch.uint8)[:, :40], tb.view(torch.uint8)[:, :40])
    with pytest.raises(TypeError):
        fn(ta.view(torch.uint8).float(), tb)
    with pytest.raises(ValueError):
        fn(ta.view(torch.uint8).cpu(), tb)
    assert BACKEND.supports(SimpleNamespace(device="cpu", fmt_a="e4m3", fmt_b="e4m3", preset="ada")) is not None


def test_launch_accounting(monkeypatch):
    from mmaemu_b200 import _lib
    monkeypatch.setenv("MMAEMU_B200_ROW_GROUPS", "0")    # the 8-row-slot kernels and their pre-decode launches
    a, b, ta, tb = operands(48, 16, 64, seed=7)
    n0 = _lib.launch_count()
    mm.accumulate(ta, tb, use_fast_accum=True, profile="ada", splitk=1)
    assert _lib.launch_count() == n0 + 3              # two pre-decode kernels and the GEMM kernel (scratch memory path)
    mm.accumulate(ta, tb, use_fast_accum=True, profile="ada", splitk=1, backend="cuda:b200-direct")
    assert _lib.launch_count() == n0 + 4              # one kernel that decodes in its main loop
    mm.accumulate(ta, tb, use_fast_accum=True, profile="ada", splitk=(2, "serial"), backend="cuda:b200")
    assert _lib.launch_count() == n0 + 8              # split plan: pre-decode x 2, the tile order, the GEMM kernel
    mm.accumulate(ta, tb, use_fast_accum=True, profile="ada", splitk=(2, "serial"), backend="cuda:b200-direct")
    assert _lib.launch_count() == n0 + 9              # without scratch memory split plans run on the integer kernel
    a, b, ta, tb = operands(48, 16, 512, seed=8)
    mm.accumulate(ta, tb, use_fast_accum=False, profile="ada", splitk=1)
    assert _lib.launch_count() == n0 + 14             # few tiles, 4 chains: pre-decode x 2, tile order, K slices, combine
    # the 16-row kernels decode both operands themselves, so the pre-decode launches disappear: calls of at most 16
    # rows always, and -- by default -- calls whose output tiles and chains would leave most SMs without a CTA
    for M, env in ((16, "0"), (48, "1")):
        monkeypatch.setenv("MMAEMU_B200_ROW_GROUPS", env)
        a, b, ta, tb = operands(M, 16, 512, seed=9)
        n0 = _lib.launch_count()
        mm.accumulate(ta, tb, use_fast_accum=True, profile="ada", splitk=1)
        assert _lib.launch_count() == n0 + 1          # the GEMM kernel alone
        mm.accumulate(ta, tb, use_fast_accum=False, profile="ada", splitk=1)
        assert _lib.launch_count() == n0 + 4          # tile order, K slices, combine
        mm.accumulate(ta, tb, use_fast_accum=True, profile="ada", splitk=(2, "serial"))
        assert _lib.launch_count() == n0 + 7          # a split plan in K slices: tile order, K slices, combine


def test_call_is_capturable_in_a_cuda_graph():
    """No host synchronisation anywhere in the call (scales and non-finite flags stay on the device), so a scaled_mm
    call can be captured once and replayed on new operand values -- the gap the reference documents for its CUDA path
    (docs/backends.md:116-117 of astding/mmaemu). The replay must equal eager calls bit for bit, also when the new
    operands hold NaN codes and when the plan is split."""
    M, N, K = 192, 256, 2048
    rng = np.random.default_rng(21)
    a0 = datagen._round_to(rng.standard_normal((M, K)) * 4, "e4m3")
    b0 = datagen._round_to(rng.standard_normal((N, K)) * 4, "e4m3")
    ta = torch.from_numpy(a0).to(DEV).view(F8["e4m3"])
    tb = torch.from_numpy(b0).to(DEV).view(F8["e4m3"])
    sa, sb = torch.tensor(0.5, device=DEV), torch.tensor(2.0, device=DEV)
    for profile, split in (("hopper", 1), ("ada", (3, "pairwise"))):
        kw = dict(out_dtype=torch.bfloat16, profile=profile, splitk=split)
        mm.scaled_mm(ta, tb.t(), sa, sb, **kw)                     # warm-up outside the capture
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            y = mm.scaled_mm(ta, tb.t(), sa, sb, **kw)
        for trial in range(3):
            a1 = datagen._round_to(rng.standard_normal((M, K)) * 4, "e4m3")
            b1 = datagen._round_to(rng.standard_normal((N, K)) * 4, "e4m3")
            if trial == 2:
                a1[5, 77] = 0x7F                                    # a NaN row
                b1[9, 3] = 0xFF                                     # and a NaN column
            ta.view(torch.uint8).copy_(torch.from_numpy(a1))
            tb.view(torch.uint8).copy_(torch.from_numpy(b1))
            sa.fill_(0.25 * (trial + 1))
            g.replay()
            torch.cuda.synchronize()
            want = oracle.scaled_mm(a1, b1, 0.25 * (trial + 1), 2.0, out="bfloat16", preset=profile, fast=False,
                                    S=1 if split == 1 else split[0], scheme="none" if split == 1 else split[1])
            assert np.array_equal(bits(y), want), (profile, trial)


@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16), ids=("fp32", "bf16"))
def test_quantised_activations(dtype):
    """quantized_scaled_mm: the E4M3 codes equal torch's (x * s).clamp(-448, 448).to(float8_e4m3fn) on the device, and
    the product equals scaled_mm on those codes (checked against the oracle), for contiguous and padded activations,
    an unsplit and a split plan; rows that are not 16-byte aligned are refused (no path through torch operations)."""
    rng = np.random.default_rng(31)
    for (M, N, K, pad, profile, split) in ((200, 192, 1024, 0, "hopper-te", 1), (64, 128, 2048, 24, "ada", (4, "serial")),
                                           (33, 48, 1008, 3, "hopper", 1)):
        x = rng.standard_normal((M, K + pad)).astype(np.float32)
        x[3, 5], x[7, 9], x[11, 2], x[13, 1] = 1e9, -np.inf, np.nan, 1e-12       # clamp, -inf, NaN, underflow
        x[1, :8] = [0.0, -0.0, 2.0 ** -20, -2.0 ** -19, 3.0, -3.0, 0.05, 100.0]
        xt = torch.from_numpy(x).to(DEV).to(dtype)[:, :K]
        finite = torch.where(torch.isfinite(xt) & (xt.abs() < 1e6), xt.abs().float(), torch.zeros((), device=DEV))
        qs = (448.0 / finite.max()).to(torch.float32)
        w = datagen._round_to(rng.standard_normal((N, K)) * 0.02 * 448 / 0.08, "e4m3")
        tw = torch.from_numpy(w).to(DEV).view(F8["e4m3"])
        sa, sb = (1.0 / qs).to(torch.float32), torch.tensor(0.08 / 448, device=DEV)
        if pad % (4 if dtype == torch.float32 else 8):
            with pytest.raises(ValueError, match="16-byte"):
                mm.quantized_scaled_mm(xt, qs, tw.t(), sa, sb, out_dtype=torch.bfloat16, profile=profile, splitk=split)
            continue
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            y, xq = mm.quantized_scaled_mm(xt, qs, tw.t(), sa, sb, out_dtype=torch.bfloat16, profile=profile,
                                           splitk=split, return_codes=True)
        want_q = (xt * qs).clamp(-448, 448).to(torch.float8_e4m3fn)
        assert torch.equal(xq.view(torch.uint8), want_q.view(torch.uint8)), (M, N, K, dtype)
        codes = xq.view(torch.uint8).cpu().numpy()
        assert codes[11, 2] == 0x7F and codes[3, 5] == 0x7E and codes[7, 9] == 0xFE and codes[13, 1] == 0x00
        S, scheme = (1, "none") if split == 1 else split
        want = oracle.scaled_mm(codes, w, float(sa), float(sb), out="bfloat16", preset=profile.split("-")[0], fast=False,
                                S=S, scheme=scheme)
        assert np.array_equal(bits(y), want), (M, N, K, dtype)


def test_quantised_activations_argument_checks():
    x = torch.zeros(16, 32, device=DEV)
    w = torch.zeros(16, 32, device=DEV).to(torch.float8_e4m3fn)
    one = torch.ones((), device=DEV)
    with pytest.raises(TypeError):
        mm.quantized_scaled_mm(x.half(), one, w.t(), one, one, out_dtype=torch.bfloat16, splitk=1)
    with pytest.raises(TypeError):
        mm.quantized_scaled_mm(x, 2.0, w.t(), one, one, out_dtype=torch.bfloat16, splitk=1)
    with pytest.raises(mm.SplitKUnknownError):                      # scaled_mm's own checks apply to the produced tensor
        mm.quantized_scaled_mm(x, one, w.t(), one, one, out_dtype=torch.bfloat16, profile="hopper")
    # rows that the decode pass cannot read with 16-byte loads: refused, never computed by torch operations instead
    wide = torch.zeros(16, 34, device=DEV)
    with pytest.raises(ValueError, match="16-byte"):
        mm.quantized_scaled_mm(wide[:, 1:33], one, w.t(), one, one, out_dtype=torch.bfloat16, splitk=1, profile="ada")
    empty = mm.quantized_scaled_mm(x[:0], one, w.t(), one, one, out_dtype=torch.bfloat16, splitk=1, profile="ada")
    assert empty.shape == (0, 16)


def test_a_wait_that_runs_out_is_reported_and_nothing_is_written(monkeypatch):
    """The scratch-memory kernels bound every wait for their bulk copies. The test hook makes the copies announce 16
    bytes more than they bring, so the barrier of the first stage never completes: the kernel must give up after the
    (shortened) bound, record the status word, leave D untouched and return -- no fault, no endless spin -- and the
    entry points that read the word must report MMB200_ERR_TIMEOUT. The next call, with the hook cleared, works."""
    L = _lib.load()
    monkeypatch.setenv("MMAEMU_B200_ROW_GROUPS", "0")   # the kernels with the ring (the 16-row kernels have no waits)
    M, N, K = 256, 128, 512
    rng = np.random.default_rng(9)
    a = torch.from_numpy(datagen.codes(rng, M, K, "e4m3", "gauss40")).to(DEV)
    b = torch.from_numpy(datagen.codes(rng, N, K, "e4m3", "gauss40")).to(DEV)
    sc = torch.tensor([0.5, 2.0], dtype=torch.float32, device=DEV)
    n = int(L.mmb200_workspace_bytes_split(M, N, K, 1))
    ws = torch.zeros(n, dtype=torch.uint8, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream(DEV).cuda_stream)

    def call(D):
        return L.mmb200_scaled_mm_ws(a.data_ptr(), K, 0, b.data_ptr(), K, 0, D.data_ptr(), N, _lib.OUT_CODES["bfloat16"],
                                     M, N, K, 32, 1, 1, 0, sc.data_ptr(), sc.data_ptr() + 4, None, 0, ws.data_ptr(), n,
                                     stream)
    L.mmb200_test_hooks(1000, 16)
    try:
        D = torch.full((M, N), 0x5555, dtype=torch.int16, device=DEV)
        assert call(D) == _lib.OK                                  # the launch itself succeeds; it is asynchronous
        assert L.mmb200_workspace_status(ws.data_ptr(), M, N, K, 1, stream) == _lib.ERR_TIMEOUT
        assert bool((D == 0x5555).all())                           # nothing was written
        off = int(L.mmb200_workspace_status_offset(M, N, K, 1))
        assert int(ws[off:off + 4].view(torch.int32).item()) == 1
        with pytest.raises(_lib.NativeError) as e:
            _lib.check("mmb200_workspace_status", _lib.ERR_TIMEOUT)
        assert e.value.status == _lib.ERR_TIMEOUT
        # the host-buffer entry point synchronises anyway and must return the error instead of a stale result
        ah, bh = a.cpu().numpy(), b.cpu().numpy()
        dh = np.full((M, N), 0x5555, dtype=np.uint16)
        rc = L.mmb200_scaled_mm_host(ah.ctypes.data, K, 0, bh.ctypes.data, K, 0, dh.ctypes.data, N,
                                     _lib.OUT_CODES["bfloat16"], M, N, K, 32, 1, 1, 0, ctypes.c_float(0.5),
                                     ctypes.c_float(2.0), None, 0, stream)
        assert rc == _lib.ERR_TIMEOUT and bool((dh == 0x5555).all())
        # the Python entry point checks the word when asked to
        os.environ["MMAEMU_B200_CHECK_STATUS"] = "1"
        with pytest.raises(_lib.NativeError):
            mm.scaled_mm(a.view(torch.float8_e4m3fn), b.view(torch.float8_e4m3fn).t(), sc[0], sc[1],
                         out_dtype=torch.bfloat16, use_fast_accum=True, profile="hopper", splitk=1)
    finally:
        os.environ.pop("MMAEMU_B200_CHECK_STATUS", None)
        L.mmb200_test_hooks(0, 0)
    D = torch.full((M, N), 0x5555, dtype=torch.int16, device=DEV)
    assert call(D) == _lib.OK
    assert L.mmb200_workspace_status(ws.data_ptr(), M, N, K, 1, stream) == _lib.OK
    want = oracle.scaled_mm(a.cpu().numpy(), b.cpu().numpy(), 0.5, 2.0, out="bfloat16", preset=32, fast=True)
    assert np.array_equal(D.cpu().numpy().view(np.uint16), want)


@pytest.mark.parametrize("pipeline", ("1", "0"))
def test_scaled_mm_host_slabs_equal_the_single_launch(pipeline, monkeypatch):
    """Host operands in, host result out (mmb200_scaled_mm_host): calls large enough to be cut into row slabs that
    overlap copies and kernels on internal streams must give the bits of the oracle and of scaled_mm on device
    tensors -- ragged last slab, NaN codes in a late slab and in B, a split-K plan of the whole call, pinned and
    pageable host memory, a padded out= -- and the same with the slabs turned off."""
    monkeypatch.setenv("MMAEMU_B200_HOST_PIPELINE", pipeline)
    M, N, K = 4200, 2048, 512                            # 33 x 16 output tiles: four slabs of 1024 rows and one of 104
    rng = np.random.default_rng(77)
    a = datagen.codes(rng, M, K, "e4m3", "gauss40")
    b = datagen.codes(rng, N, K, "e4m3", "all_codes")
    a[4150, 17], a[100, 3], b[2000, 500] = 0x7F, 0xFF, 0x7F
    ta, tb = torch.from_numpy(a).view(F8["e4m3"]), torch.from_numpy(b).view(F8["e4m3"])
    sa, sb = torch.tensor(0.75), torch.tensor(1.5)
    want = oracle.scaled_mm(a, b, 0.75, 1.5, out="bfloat16", preset="hopper", fast=False)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        y = mm.scaled_mm_host(ta.pin_memory(), tb.pin_memory().t(), sa, sb, out_dtype=torch.bfloat16, profile="hopper",
                              splitk=1)
        assert y.device.type == "cpu" and np.array_equal(bits(y), want)
        y = mm.scaled_mm_host(ta, tb.t(), sa, sb, out_dtype=torch.bfloat16, profile="hopper", splitk=1)   # pageable
        assert np.array_equal(bits(y), want)
        # a split-K plan (decided for the whole call, handed to every slab), fp8 output with scale_result, out= with a
        # padded leading dimension, and twice in a row (the staging pool and the internal streams are reused)
        sr = torch.tensor(0.5)
        big = torch.zeros((M, N + 64), dtype=torch.float8_e4m3fn).pin_memory()
        dev_y = mm.scaled_mm(ta.to(DEV), tb.to(DEV).t(), sa.to(DEV), sb.to(DEV), scale_result=sr.to(DEV),
                             out_dtype=torch.float8_e4m3fn, use_fast_accum=True, profile="hopper",
                             splitk=(2, "contiguous"))
        for _ in range(2):
            out = mm.scaled_mm_host(ta.pin_memory(), tb.pin_memory().t(), sa, sb, scale_result=sr,
                                    out_dtype=torch.float8_e4m3fn, use_fast_accum=True, profile="hopper",
                                    splitk=(2, "contiguous"), out=big[:, :N])
            assert out.data_ptr() == big.data_ptr() and np.array_equal(bits(out), bits(dev_y))
        assert not big[:, N:].view(torch.uint8).any()
        # formats and presets the staged kernels do not serve take the one-launch path of the same entry point
        a5 = datagen.codes(rng, 300, 192, "e5m2", "gauss40")
        y = mm.scaled_mm_host(torch.from_numpy(a5).view(F8["e5m2"]), tb[:160, :192].t(), sa, sb,
                              out_dtype=torch.float16, use_fast_accum=True, profile="b200-mma-sync-experimental", splitk=1)
    assert np.array_equal(bits(y), oracle.scaled_mm(a5, b[:160, :192], 0.75, 1.5, out="float16", fmt_a="e5m2",
                                                    preset=288, fast=True))
