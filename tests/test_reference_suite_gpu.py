"""The reference's own GPU test files, run unchanged with the B200 backend selected through install_into_reference()
(-m gpu). Only the backend name differs from what the reference's authors run:

  * tests/test_hw_mini.py::test_gpu_backend    the 2,519 recorded RTX 4060 cases (astding/mmaemu tests/test_hw_mini.py:323);
  * tests/test_h100_mini.py::_run              the recorded H100 PCIe calls, by sha256 of the hardware output
                                               (tests/test_h100_mini.py:52-83), for the format pair its explicit-kernel
                                               cases use;
  * tests/test_kernels_ieee.py                 the kernel conformance data (8 classes x 48 shapes, :34-36), slow
                                               accumulation, every split layout and ragged K, with the module's kernel
                                               factory `_chain` returning this backend's ChainFn for the kernel's preset.

The reference package, its tests and their data are taken from baseline/_ref/ (baseline/install_reference.py); the
test modules are imported from there by file path and their functions are called directly.
"""
import importlib.util
import sys
import warnings
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT / "baseline"))
import install_reference  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)
REF_TESTS = install_reference.DEST / "tests"


@pytest.fixture(scope="module")
def ref():
    if not install_reference.add_to_path() or not (REF_TESTS / "test_hw_mini.py").exists():
        pytest.skip("the reference package and its tests are not installed under baseline/_ref "
                    "(python baseline/install_reference.py)")
    import mmaemu
    from mmaemu_b200 import backend as b200
    b200.install_into_reference()
    yield mmaemu
    b200.uninstall_from_reference()


def load(name):
    """A test module of the reference, imported from baseline/_ref/tests by path (its conftest is not involved)."""
    path = REF_TESTS / f"{name}.py"
    spec = importlib.util.spec_from_file_location(f"reference_{name}", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


def test_hw_mini_gpu_backend(ref, capsys):
    mod = load("test_hw_mini")
    mod.GPU_BACKENDS = tuple(mod.GPU_BACKENDS) + ("cuda:b200",)
    st = ref.backends_status(DEV)
    assert st["cuda:b200"].available, st["cuda:b200"].reason
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        mod.test_gpu_backend("cuda:b200")
    out = capsys.readouterr().out
    print(out)
    assert "backend cuda:b200:" in out and " 0 failed" in out


def test_h100_mini_jobs(ref):
    mod = load("test_h100_mini")
    jobs = [j for j in mod.JOBS if (j["fa"], j["fb"]) == ("e4m3", "e4m3")]
    assert len(jobs) > 20
    for j in jobs:
        mod._run(j, DEV, "cuda:b200")


@pytest.fixture(scope="module")
def ieee(ref, tmp_path_factory):
    import os
    os.environ["MMAEMU_TEST_REF_CACHE"] = str(tmp_path_factory.mktemp("ieee_refs"))
    mod = load("test_kernels_ieee")
    from mmaemu.backends import ChainRequest
    from mmaemu_b200.backend import BACKEND

    def chain(spec, dev):
        return BACKEND.chain_fn(ChainRequest(device=torch.device(dev), fmt_a="e4m3", fmt_b="e4m3", preset=spec.preset))
    mod._chain = chain
    return mod


@pytest.mark.parametrize("kernel", ["v4", "h4"])
def test_kernels_ieee_conformance(ieee, kernel):
    """The body of test_conformance (tests/test_kernels_ieee.py:212-231) for one kernel name: all 384 cases against the
    CPU reference of the kernel's preset."""
    spec = ieee._spec(kernel)
    fn = ieee._chain(spec, DEV)
    torch.set_num_threads(max(1, (torch.get_num_threads())))
    bad, total = [], 0
    for case in ieee.CASES:
        a, b = ieee.make(*case)
        got = ieee._bits(fn(a.to(DEV), b.to(DEV)))
        want = ieee.cached_reference(case, spec.preset).view(torch.int32)
        total += want.numel()
        n = int((got != want).sum())
        if n:
            bad.append((case, n))
    assert not bad, f"{kernel}: {len(bad)} of {len(ieee.CASES)} cases differ, first {bad[:5]}"
    assert total == sum(M * N for _, M, N, _ in ieee.CASES)


@pytest.mark.parametrize("kernel", ["v4", "h4"])
def test_kernels_ieee_plans(ieee, kernel):
    """Slow accumulation, NaN codes through the plan, split-K in every layout the reference tests, ragged K and byte
    values that never fault: the reference's test functions, called with their own parameter lists."""
    for K in (1920, 8192):
        ieee.test_slow_accumulation(DEV, kernel, K)
    for fast in (True, False):
        ieee.test_nan_through_plan(DEV, kernel, fast)
    if kernel == "v4":
        for S, scheme, fast in ieee.SPLITS:
            ieee.test_split_k(DEV, kernel, S, scheme, fast)
    else:
        for S, K, fast in ieee.SPLITS_H:
            ieee.test_split_k_contiguous_hopper(DEV, kernel, S, K, fast)
    for fill in ("0xFF", "0x7F", "0x80", "uniform256"):
        ieee.test_any_byte_value_never_faults(DEV, kernel, fill)
