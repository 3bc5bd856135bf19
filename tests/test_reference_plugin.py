"""install_into_reference(): the B200 backend inside the reference's own backend selection, on a machine without a GPU.

The unmodified reference package is taken from baseline/_ref/ (baseline/install_reference.py). The selection logic is
driven the way the reference's own selection tests drive it (astding/mmaemu tests/test_backend_selection.py:34-59):
device capability and availability are programmed, no driver is touched."""
import sys
import warnings
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT / "baseline"))
import install_reference  # noqa: E402

from mmaemu_b200 import backend as b200  # noqa: E402
from oracle import oracle  # noqa: E402

E4M3 = torch.float8_e4m3fn


@pytest.fixture
def ref():
    if not install_reference.add_to_path():
        pytest.skip("the reference package is not installed under baseline/_ref (python baseline/install_reference.py)")
    import mmaemu
    from mmaemu.backends import registry
    registry.clear()
    b200.install_into_reference()
    yield mmaemu
    b200.uninstall_from_reference()
    registry.clear()


def operands(M=32, N=48, K=64):
    g = torch.Generator().manual_seed(1)
    a = (torch.randn(M, K, generator=g) * 4).to(E4M3)
    bt = (torch.randn(N, K, generator=g) * 4).to(E4M3)
    return a, bt


def test_install_is_idempotent_and_extends_the_names(ref):
    from mmaemu import backends
    from mmaemu.backends import registry
    first = registry.select
    assert b200.install_into_reference() is registry and registry.select is first
    for name in ("cuda:b200", "cuda:b200-integer", "cuda:b200-fast"):
        assert backends.BACKEND_NAMES.count(name) == 1
    b200.uninstall_from_reference()
    assert "cuda:b200" not in backends.BACKEND_NAMES and registry.select is not first
    b200.install_into_reference()


def test_cpu_tensors(ref):
    """An explicit cuda:b200 on CPU tensors raises the reference's BackendUnavailableError (there is no CPU fallback);
    'auto' on CPU tensors still runs the reference's float64 model, and unknown names keep the reference's ValueError."""
    a, bt = operands()
    sa, sb = torch.tensor(0.5), torch.tensor(2.0)
    kw = dict(out_dtype=torch.bfloat16, profile="ada", splitk=1)
    with pytest.raises(ref.BackendUnavailableError) as e:
        ref.scaled_mm(a, bt.t(), sa, sb, backend="cuda:b200", **kw)
    assert type(e.value) is ref.BackendUnavailableError and "CUDA device" in str(e.value)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        y = ref.scaled_mm(a, bt.t(), sa, sb, backend="auto", **kw)
    want = oracle.scaled_mm(a.view(torch.uint8).numpy(), bt.view(torch.uint8).numpy(), 0.5, 2.0, out="bfloat16",
                            preset="ada", fast=False)
    assert np.array_equal(y.view(torch.int16).numpy().view(np.uint16), want)
    with pytest.raises(ValueError):
        ref.scaled_mm(a, bt.t(), sa, sb, backend="b200", **kw)
    cp = ref.explain(a, bt.t(), sa, sb, backend="cuda:b200", **kw)
    assert cp.validation[0] == "BackendUnavailableError"


def test_selection_on_a_programmed_device(ref, monkeypatch):
    """'auto', 'cuda' and the explicit names return the B200 backend when it supports the request; a request it does
    not support falls through to the reference's own rules ('auto') or raises (explicit name)."""
    from mmaemu.backends import ChainRequest, registry
    seen = []

    def supports(self, req):
        seen.append((self.name, req.preset))
        return None if req.preset == "hopper" else f"{self.name}: programmed refusal"
    monkeypatch.setattr(b200.B200Backend, "supports", supports)
    req = ChainRequest(device=torch.device("cuda", 0), fmt_a="e5m2", fmt_b="e4m3", preset="hopper")
    for name in ("auto", "cuda", "cuda:b200"):
        assert registry.select(req, name) is b200.BACKEND
    assert registry.select(req, "cuda:b200-integer").kernel == "integer"
    monkeypatch.setenv("MMAEMU_BACKEND", "cuda:b200-fast")
    assert registry.select(req, "auto").kernel == "fast"
    monkeypatch.delenv("MMAEMU_BACKEND")
    assert registry.explain_selection(req, "cuda:b200") == (b200.BACKEND, [])
    # refused: the explicit name raises, 'auto' falls through (no CUDA device here: the reference backend)
    other = ChainRequest(device=torch.device("cuda", 0), fmt_a="e4m3", fmt_b="e4m3", preset="ada")
    with pytest.raises(ref.BackendUnavailableError):
        registry.select(other, "cuda:b200")
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    assert registry.select(other, "auto").name == "reference"
    assert registry.select(req, "reference").name == "reference"
    assert ("cuda:b200", "hopper") in seen


def test_status_lists_the_backend(ref):
    st = ref.backends_status("cpu")
    assert "cuda:b200" in st and "reference" in st
    assert st["cuda:b200"].available is False and "CUDA device" in st["cuda:b200"].reason
