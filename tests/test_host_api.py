"""Host-side behaviour of mmaemu_b200.scaled_mm / accumulate / explain on CPU tensors (no GPU, no kernel launch):
the signature, every rejection with its exact exception class, the validation order, zero-size results, split-K
resolution and the backend names -- the contract of the reference's tests/test_api.py for this path."""
import inspect
import warnings

import pytest
import torch

import mmaemu_b200 as mm
from mmaemu_b200 import api

E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2


def ops(M=32, N=48, K=64, da=E4, db=E4):
    a = torch.zeros(M, K).to(da)
    b = torch.zeros(N, K).to(db)
    return a, b.t(), torch.tensor(1.0), torch.tensor(1.0)


def raises_exactly(cls, *args, **kw):
    with pytest.raises(cls) as ei:
        mm.scaled_mm(*args, **kw)
    assert type(ei.value) is cls, type(ei.value)
    return ei.value


def test_signature_is_torch_scaled_mm_plus_keywords():
    sig = inspect.signature(mm.scaled_mm)
    names = list(sig.parameters)
    assert names == ["input", "mat2", "scale_a", "scale_b", "bias", "scale_result", "out_dtype", "use_fast_accum", "out",
                     "profile", "splitk", "backend"]
    p = sig.parameters
    assert p["use_fast_accum"].default is False and p["out_dtype"].default is None and p["bias"].default is None
    assert p["splitk"].default == "auto" and p["backend"].default == "auto" and p["profile"].default is None
    assert all(p[n].kind is inspect.Parameter.KEYWORD_ONLY for n in ("out", "profile", "splitk", "backend"))
    assert inspect.signature(mm.explain).parameters.keys() == sig.parameters.keys()
    acc = inspect.signature(mm.accumulate).parameters
    assert acc["use_fast_accum"].default is inspect.Parameter.empty


def test_argument_types():
    a, bt, s, _ = ops()
    raises_exactly(TypeError, a.float().numpy(), bt, s, s)
    raises_exactly(TypeError, a, bt, 1.0, s)
    raises_exactly(TypeError, a, bt, s, s, bias=1.0)
    raises_exactly(TypeError, a, bt, s, s, out_dtype="bfloat16")
    raises_exactly(TypeError, a, bt, s, s, use_fast_accum=1)
    raises_exactly(TypeError, a, bt, s, s, out=3)


@pytest.mark.parametrize("make,kw", [
    (lambda: (torch.zeros(32).to(E4), ops()[1]), {}),
    (lambda: (ops()[0], torch.zeros(48, 48).to(E4).t()), {}),                            # inner dimensions differ
    (lambda: (ops()[0].float(), ops()[1]), {}),                                          # not float8
    (lambda: (ops(da=E5)[0], ops(db=E5)[1]), {}),                                        # e5m2 x e5m2
    (lambda: (ops(K=72)[0], ops(K=72)[1]), {}),                                          # K % 16
    (lambda: (ops()[0], ops(N=40)[1]), {}),                                              # N % 16
    (lambda: ops()[:2], dict(out_dtype=torch.float32, out=torch.zeros(32, 48, dtype=torch.bfloat16))),
    (lambda: ops()[:2], dict(scale_result=torch.tensor([1.0, 2.0]))),
    (lambda: ops()[:2], dict(bias=torch.zeros(7, dtype=torch.bfloat16), out_dtype=torch.bfloat16)),
    (lambda: ops()[:2], dict(bias=torch.zeros(48, dtype=torch.bfloat16), out_dtype=torch.float32)),
    (lambda: ops()[:2], dict(out_dtype=torch.float64)),
    (lambda: ops()[:2], dict(out_dtype=E5)),                                             # profile reject e4m3^2 -> e5m2
    (lambda: (ops()[0].t().contiguous().t(), ops()[1]), {}),                             # column-major mat1
    (lambda: (ops()[0], torch.zeros(64, 48).to(E4)), {}),                                # row-major mat2
])
def test_reference_rejects(make, kw):
    a, bt = make()
    kw.setdefault("out_dtype", torch.bfloat16)
    raises_exactly(mm.ReferenceRejectsError, a, bt, torch.tensor(1.0), torch.tensor(1.0), profile="ada", **kw)


def test_scale_checks():
    a, bt, s, _ = ops()
    raises_exactly(mm.ReferenceRejectsError, a, bt, s.double(), s, out_dtype=torch.bfloat16)
    raises_exactly(mm.ReferenceRejectsError, a, bt, torch.ones(32), torch.ones(48), out_dtype=torch.bfloat16)
    raises_exactly(mm.ReferenceRejectsError, a, bt, torch.ones(32, 2), torch.ones(2, 48), out_dtype=torch.bfloat16)
    raises_exactly(mm.ReferenceRejectsError, a, bt, torch.ones(32, 1), torch.ones(1, 48), out_dtype=torch.float16)


def test_scope_raises_unsupported_feature():
    a, bt, s, _ = ops()
    kw = dict(out_dtype=torch.bfloat16, profile="ada")
    raises_exactly(mm.UnsupportedFeatureError, a, bt, s, s, torch.zeros(48, dtype=torch.bfloat16), **kw)   # positional
    raises_exactly(mm.UnsupportedFeatureError, a, bt, s, s, bias=torch.zeros(48, dtype=torch.bfloat16), **kw)
    raises_exactly(mm.UnsupportedFeatureError, a, bt, torch.ones(32, 1), torch.ones(1, 48), **kw)
    sg = torch.tensor(1.0, requires_grad=True)
    raises_exactly(mm.UnsupportedFeatureError, a, bt, sg, s, **kw)
    with torch.no_grad():
        raises_exactly(mm.BackendUnavailableError, a, bt, sg, s, **kw)          # valid: only the device is missing


def test_validation_order():
    a, bt, s, _ = ops()
    bias = torch.zeros(48, dtype=torch.bfloat16)
    # a torch-level rejection wins over the scope error, the scope error over split-K, split-K over the backend
    raises_exactly(mm.ReferenceRejectsError, a, bt, s, s, bias=bias, out_dtype=torch.float32, profile="ada")
    raises_exactly(mm.UnsupportedFeatureError, a, bt, s, s, bias=bias, out_dtype=torch.bfloat16, profile="hopper")
    raises_exactly(mm.SplitKUnknownError, a, bt, s, s, out_dtype=torch.bfloat16, profile="hopper")
    raises_exactly(mm.BackendUnavailableError, a, bt, s, s, out_dtype=torch.bfloat16, profile="hopper", splitk=1)
    raises_exactly(ValueError, a, bt, s, s, out_dtype=torch.bfloat16, profile="ada", splitk=3)
    raises_exactly(ValueError, a, bt, s, s, out_dtype=torch.bfloat16, profile="ada", backend="nope")
    raises_exactly(mm.BackendUnavailableError, a, bt, s, s, out_dtype=torch.bfloat16, profile="ada", backend="cuda:h4")
    raises_exactly(mm.BackendUnavailableError, a, bt, s, s, out_dtype=torch.bfloat16, profile="ada", backend="reference")


def test_zero_sizes_return_before_the_cublas_checks():
    s = torch.tensor(1.0)
    for M, N, K in ((0, 48, 64), (32, 0, 64), (32, 48, 0)):
        a, bt, _, _ = ops(M, N, K)
        for od in (torch.float32, torch.bfloat16, E5):
            y = mm.scaled_mm(a, bt, s, s, out_dtype=od)
            assert y.shape == (M, N) and y.dtype == od and not bool(y.float().any())
    fn = getattr(torch, "float8_e4m3fnuz", None)
    if fn is not None:                                                     # accepted by torch before its early return
        assert mm.scaled_mm(torch.zeros(0, 64).to(fn), torch.zeros(48, 64).to(fn).t(), s, s).shape == (0, 48)
    assert mm.accumulate(torch.zeros(0, 8).to(E4), torch.zeros(3, 8).to(E4), use_fast_accum=True).shape == (0, 3)


def test_explain_reports_instead_of_raising():
    a, bt, s, _ = ops()
    cp = mm.explain(a, bt, s, s, out_dtype=torch.bfloat16, profile="ada")
    assert cp.validation == "ok" and (cp.profile, cp.preset, cp.preset_maturity) == ("ada", "ada", "validated")
    assert (cp.split.S, cp.split.source) == (1, "table") and cp.backend == "cuda:b200"
    cp = mm.explain(a, bt, s, s, out_dtype=torch.bfloat16)
    assert cp.validation[0] == "SplitKUnknownError" and cp.profile == "hopper"
    cp = mm.explain(a, bt, s, s, out_dtype=torch.bfloat16, profile="ada", splitk=(2, "contiguous"))
    assert cp.validation[0] == "ValueError"
    cp = mm.explain(a, bt, s, s, out_dtype=torch.bfloat16, profile="hopper", splitk=(2, "contiguous"),
                    backend="cuda:b200-integer")
    assert cp.validation == "ok" and cp.backend == "cuda:b200-integer" and cp.warnings
    assert mm.explain(a[:, :0], bt[:0], s, s).backend.startswith("none")


def test_column_major_out_swaps_the_split_key(monkeypatch):
    seen = {}

    def fake(M, N, K, **kw):
        seen.update(M=M, N=N, a=kw["a_dtype"], b=kw["b_dtype"])
        raise mm.SplitKUnknownError("stop")
    monkeypatch.setattr(api, "resolve_splitk", fake)
    a, bt, s, _ = ops(32, 48, 64, E4, E5)
    with pytest.raises(mm.SplitKUnknownError):
        mm.scaled_mm(a, bt, s, s, out=torch.zeros(48, 32).t(), profile="ada")
    assert seen == dict(M=48, N=32, a=E5, b=E4)
    with pytest.raises(mm.SplitKUnknownError):
        mm.scaled_mm(a, bt, s, s, out=torch.zeros(32, 48), profile="ada")
    assert seen == dict(M=32, N=48, a=E4, b=E5)


def test_profiles_and_env(monkeypatch):
    assert mm.list_profiles()[:6] == ["ada", "ada-te", "ada-ws0", "hopper", "hopper-te", "hopper-ws0"]
    assert mm.get_profile().name == "hopper"
    monkeypatch.setenv("MMAEMU_PROFILE", "ada-te")
    assert mm.get_profile().name == "ada-te" and mm.get_profile().workspace_bytes == 4 << 20
    with pytest.raises(KeyError):
        mm.get_profile("h100")
    a, bt, s, _ = ops()
    with pytest.warns(mm.ExperimentalPresetWarning):
        with pytest.raises(mm.SplitKUnknownError):
            mm.scaled_mm(a, bt, s, s, out_dtype=torch.bfloat16, profile="hopper-experimental")
    monkeypatch.setenv("MMAEMU_BACKEND", "cuda:v4")
    with pytest.raises(mm.BackendUnavailableError):
        mm.scaled_mm(a, bt, s, s, out_dtype=torch.bfloat16, profile="ada")


def test_accumulate_argument_checks():
    a, b = torch.zeros(4, 16).to(E4), torch.zeros(5, 16).to(E4)
    with pytest.raises(TypeError):
        mm.accumulate(a, b)                                                   # use_fast_accum has no default
    with pytest.raises(TypeError):
        mm.accumulate(a, b, use_fast_accum=1)
    with pytest.raises(TypeError):
        mm.accumulate(a.float(), b, use_fast_accum=True)
    with pytest.raises(ValueError):
        mm.accumulate(a, b[:, :8], use_fast_accum=True)
    with pytest.raises(mm.BackendUnavailableError):
        mm.accumulate(a, b, use_fast_accum=True, profile="ada", splitk=1)


def test_presets():
    from mmaemu_b200.numerics import check_plan, get_preset
    assert (get_preset("ada").nfma, get_preset("hopper").nfma) == (16, 32)
    with pytest.raises(KeyError):
        get_preset("volta")
    # the late-accumulator preset (mmaemu/model/presets.py:78-85, alias 'blackwell'): fast, unsplit plans only
    late = get_preset("b200_mma_sync")
    assert (late.nfma, late.frac, late.frac_out, late.min_exp, late.late_c, late.slow_chunk, late.maturity, late.code) == (
        32, 25, 23, -133, True, None, "experimental", 288)
    assert (get_preset("ada").code, get_preset("hopper").code) == (16, 32)
    assert check_plan(late, 4096, 1, "none", True) == "none"
    with pytest.raises(mm.UnsupportedFeatureError, match="slow accumulation"):
        check_plan(late, 4096, 1, "none", False)
    with pytest.raises(mm.UnsupportedFeatureError, match="split-K"):
        check_plan(late, 4096, 2, "contiguous", True)
    from mmaemu_b200 import numerics
    numerics._reset_warnings_for_tests()
    with pytest.warns(mm.ExperimentalPresetWarning, match="NOT B200 cuBLAS"):
        assert get_preset("b200_mma_sync", warn=True) is late
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        get_preset("b200_mma_sync", warn=True)                                # once per name
    for _ in range(2):                                                        # the alias warns on every lookup
        with pytest.warns(mm.ExperimentalPresetWarning, match="alias of 'b200_mma_sync'"):
            assert get_preset("blackwell", warn=True) is late

    class Foreign:                                                            # e.g. the reference's own Preset object
        name, nfma, frac, frac_out, min_exp, late_c, slow_chunk = "b200_mma_sync", 32, 25, 23, -133, True, None
    assert get_preset(Foreign()) is late
    Foreign.frac = 20
    with pytest.raises(mm.UnsupportedFeatureError):
        get_preset(Foreign())
    prof = mm.get_profile("b200-mma-sync-experimental")
    assert (prof.preset, prof.capability, prof.splitk_table, prof.maturity) == ("b200_mma_sync", (10, 0), None, "experimental")
    assert check_plan(get_preset("ada"), 64, 1, "pairwise") == "none"
    assert check_plan(get_preset("hopper"), 64, 4, "contiguous") == "contiguous"
    for bad in ((get_preset("ada"), 4, "contiguous"), (get_preset("hopper"), 2, "serial"), (get_preset("ada"), 2, "x")):
        with pytest.raises(ValueError):
            check_plan(bad[0], 64, bad[1], bad[2])


def test_scaled_mm_host_validates_like_scaled_mm():
    """The host-buffer entry point checks the call from metadata in scaled_mm's order before it touches a device."""
    a, bt, sa, sb = ops()
    assert "scaled_mm_host" in mm.__all__
    y = mm.scaled_mm_host(a[:0], bt, sa, sb, out_dtype=torch.bfloat16)                 # zero-size result: no device needed
    assert y.shape == (0, 48) and y.dtype == torch.bfloat16
    y = mm.scaled_mm_host(a[:, :0], bt[:0], sa, sb, out_dtype=torch.float16)           # K == 0: +0 everywhere
    assert y.shape == (32, 48) and not y.any()
    with pytest.raises(mm.ReferenceRejectsError):
        mm.scaled_mm_host(a.to(E5), bt.to(E5), sa, sb, out_dtype=torch.bfloat16, splitk=1)
    with pytest.raises(mm.ReferenceRejectsError):
        mm.scaled_mm_host(a, bt.t().contiguous().t().contiguous(), sa, sb, out_dtype=torch.bfloat16, splitk=1)   # row-major mat2
    with pytest.raises(mm.UnsupportedFeatureError):
        mm.scaled_mm_host(a, bt, torch.full((32, 1), 1.0), torch.full((1, 48), 1.0), out_dtype=torch.bfloat16)
    with pytest.raises(mm.SplitKUnknownError):
        mm.scaled_mm_host(a, bt, sa, sb, out_dtype=torch.bfloat16, profile="hopper-experimental")
    with pytest.raises(ValueError, match="out must be"):
        mm.scaled_mm_host(a, bt, sa, sb, out_dtype=torch.bfloat16, splitk=1, out=torch.empty(32, 47, dtype=torch.bfloat16))
    with pytest.raises(mm.UnsupportedFeatureError, match="slow accumulation"):
        mm.scaled_mm_host(a, bt, sa, sb, out_dtype=torch.bfloat16, splitk=1, profile="b200-mma-sync-experimental")
    if not torch.cuda.is_available():
        with pytest.raises(mm.BackendUnavailableError):
            mm.scaled_mm_host(a, bt, sa, sb, out_dtype=torch.bfloat16, splitk=1)
