"""The C-ABI library loads on a machine without a GPU and exports every function include/mmaemu_b200.h declares; calls
that need a device fail with a status, never with a crash. No kernel is launched here."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
HEADER = (ROOT / "include" / "mmaemu_b200.h").read_text()


def declared_functions():
    code = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
    return sorted(set(re.findall(r"\b(mmb200_[a-z0-9_]+)\s*\(", code)))


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as entry
    entry.build()
    from mmaemu_b200 import _lib
    return _lib.load()


def test_header_declares_the_expected_entry_points():
    from mmaemu_b200 import _lib
    assert set(declared_functions()) == set(_lib.EXPORTS)


def test_every_declared_function_is_exported(lib):
    for name in declared_functions():
        assert hasattr(lib, name), name


def test_status_codes_and_argument_checks_without_a_device(lib):
    from mmaemu_b200 import _lib
    assert lib.mmb200_abi_version() == int(re.search(r"#define MMB200_ABI_VERSION (\d+)", HEADER).group(1))
    for code in (0, -1, -2, -3, -4, -5, -6):
        assert lib.mmb200_status_string(code).decode() not in ("", "unknown status")
    assert lib.mmb200_status_string(-99).decode() == "unknown status"
    buf = ctypes.create_string_buffer(64)
    p = ctypes.addressof(buf)
    # argument errors are reported before any CUDA call
    assert lib.mmb200_chain(p, 16, 7, p, 16, 0, p, 1, 1, 1, 16, 32, 0, None) == _lib.ERR_BAD_ARG      # bad format
    assert lib.mmb200_chain(p, 8, 0, p, 16, 0, p, 1, 1, 1, 16, 32, 0, None) == _lib.ERR_BAD_ARG       # lda < K
    assert lib.mmb200_chain(p, 16, 0, p, 16, 0, p, 1, 1, 1, 16, 24, 0, None) == _lib.ERR_UNSUPPORTED  # nfma
    assert lib.mmb200_accumulate(p, 16, 0, p, 16, 0, p, 1, 1, 1, 16, 32, 1, 2, 0, 0, None) == _lib.ERR_BAD_ARG
    assert lib.mmb200_accumulate(p, 16, 0, p, 16, 0, p, 1, 1, 1, 16, 32, 1, 65, 3, 0, None) == _lib.ERR_TOO_LARGE
    assert lib.mmb200_scaled_mm(p, 16, 0, p, 16, 0, p, 1, 1, 1, 1, 16, 32, 1, 1, 0, None, None, None, 0, None) \
        == _lib.ERR_BAD_ARG                                                                            # no scales
    assert lib.mmb200_chain(p, 16, 0, p, 16, 0, p, 1, 0, 5, 16, 32, 0, None) == _lib.OK               # empty result
    # the entry point without allocation validates before it looks at sizes or the device, as the others do
    s = p + 32
    assert lib.mmb200_scaled_mm_static(p, 16, 7, p, 16, 0, p, 16, 1, 0, 16, 16, 32, 1, s, s, None, None) == _lib.ERR_BAD_ARG
    assert lib.mmb200_scaled_mm_static(p, 16, 0, p, 16, 0, p, 16, 9, 0, 16, 16, 32, 1, s, s, None, None) == _lib.ERR_BAD_ARG
    assert lib.mmb200_scaled_mm_static(p, 16, 0, p, 16, 0, p, 16, 1, 0, 16, 16, 32, 1, None, s, None, None) == _lib.ERR_BAD_ARG
    assert lib.mmb200_scaled_mm_static(p, 16, 0, p, 16, 0, p, 16, 1, 0, 16, 16, 32, 1, s, s, None, None) == _lib.OK
    # the status word of the scratch-memory kernels: where it lives, and argument checks of its reader
    off = lib.mmb200_workspace_status_offset(4096, 4096, 4096, 1)
    assert 0 < off < lib.mmb200_workspace_bytes(4096, 4096, 4096) and off % 4 == 0
    assert off == lib.mmb200_workspace_status_offset(4096, 4096, 4096, 4)      # a prefix shared by every layout
    assert lib.mmb200_workspace_status(None, 16, 16, 16, 1, None) == _lib.OK    # no scratch memory: nothing to report
    assert lib.mmb200_workspace_status(p, -1, 16, 16, 1, None) == _lib.ERR_BAD_ARG
    assert lib.mmb200_launch_count() == 0


def test_no_device_is_a_status_not_a_crash(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from mmaemu_b200 import _lib
    buf = ctypes.create_string_buffer(64)
    p = ctypes.addressof(buf)
    rc = lib.mmb200_chain(p, 16, 0, p, 16, 0, p, 1, 1, 1, 16, 32, 0, None)
    assert rc in (_lib.ERR_LAUNCH, _lib.ERR_ARCH)
    with pytest.raises(Exception):
        _lib.check("mmb200_chain", rc)
    # the entry point without allocation records the CUDA error text when it cannot reach a device
    s = p + 32
    rc = lib.mmb200_scaled_mm_static(p, 16, 0, p, 16, 0, p, 16, 1, 16, 16, 16, 32, 1, s, s, None, None)
    assert rc in (_lib.ERR_LAUNCH, _lib.ERR_ARCH)
    if rc == _lib.ERR_LAUNCH:
        assert lib.mmb200_last_cuda_error().decode() != ""


def test_preset_numbers_of_the_header_match_the_python_presets():
    """The `nfma` argument names the preset: the header's MMB200_PRESET_* values are Preset.code of numerics.py."""
    import re
    from pathlib import Path
    from mmaemu_b200.numerics import PRESETS
    text = (Path(__file__).resolve().parents[1] / "include" / "mmaemu_b200.h").read_text()
    header = {m.group(1).lower(): int(m.group(2)) for m in re.finditer(r"#define MMB200_PRESET_(\w+) (\d+)", text)}
    assert header == {name: p.code for name, p in PRESETS.items()} == {"ada": 16, "hopper": 32, "b200_mma_sync": 288}
