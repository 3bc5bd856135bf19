"""mmb200_scaled_mm_static on a B200: the entry point for hosts that can neither allocate device memory nor lend any.

It must give the bits of the regular entry point (mmb200_scaled_mm) while taking its scratch memory from the fixed
array inside the library. Two calls in a row share that array, so the second one runs on whatever the first left
behind: it uses a smaller shape with other formats and non-finite inputs, which only comes out right if every call
clears what must start at zero. Requests beyond the array's size, or that the scratch-memory kernel does not serve,
must be refused with a status. This file is collected last on purpose (pytest --collect-only)."""
import ctypes

import numpy as np
import pytest
import torch

import datagen
from mmaemu_b200 import _lib
from oracle import oracle

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
OUT_T = {"bfloat16": torch.int16, "float32": torch.int32, "float8_e4m3fn": torch.uint8}


def call(entry, a, b, fa, fb, out, nfma, fast, scales):
    L = _lib.load()
    M, K = a.shape
    N = b.shape[0]
    A, B = torch.from_numpy(a).to(DEV), torch.from_numpy(b).to(DEV)
    D = torch.full((M, N), 0x55, dtype=torch.uint8, device=DEV).repeat(1, torch.zeros((), dtype=OUT_T[out]).element_size()) \
        .view(OUT_T[out])
    sc = torch.tensor(scales, dtype=torch.float32, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream(DEV).cuda_stream)
    sr = sc.data_ptr() + 8 if out.startswith("float8") else None
    args = [A.data_ptr(), K, _lib.FMT_CODES[fa], B.data_ptr(), K, _lib.FMT_CODES[fb], D.data_ptr(), N, _lib.OUT_CODES[out],
            M, N, K, nfma, int(fast)]
    if entry == "static":
        rc = L.mmb200_scaled_mm_static(*args, sc.data_ptr(), sc.data_ptr() + 4, sr, stream)
    else:
        rc = L.mmb200_scaled_mm(*args, 1, 0, sc.data_ptr(), sc.data_ptr() + 4, sr, _lib.KERNEL_CODES["auto"], stream)
    torch.cuda.synchronize(DEV)
    return rc, D.cpu().numpy()


def test_static_scratch_entry_point_matches_the_regular_one_twice_in_a_row():
    rng = np.random.default_rng(77)
    # first call: fills most of the array (about 43 of 64 MiB)
    a1 = datagen.codes(rng, 1024, 2304, "e4m3", "gauss40")
    b1 = datagen.codes(rng, 1024, 2304, "e4m3", "block_exponents")
    # second call: smaller, other formats, NaN and Inf codes in rows whose flags the first call left at zero or not
    a2 = datagen.codes(rng, 200, 528, "e5m2", "gauss40")
    b2 = datagen.codes(rng, 136, 528, "e4m3", "all_codes")
    a2[3, 17], a2[150, 0], b2[7, 99] = 0x7E, 0xFC, 0x7F
    first = ("e4m3", "e4m3", "bfloat16", 32, False, [0.37, 1.5, 1.0])
    second = ("e5m2", "e4m3", "float8_e4m3fn", 16, True, [0.011, 2.0, 0.75])
    L = _lib.load()
    for a, b, cfg in ((a1, b1, first), (a2, b2, second)):
        rc, got = call("static", a, b, *cfg)
        _lib.check("mmb200_scaled_mm_static", rc)
        rc, want = call("regular", a, b, *cfg)
        _lib.check("mmb200_scaled_mm", rc)
        assert np.array_equal(got, want), f"{int((got != want).sum())} of {want.size} outputs differ"
        fa, fb, out, nfma, fast, sc = cfg
        truth = oracle.scaled_mm(a, b, sc[0], sc[1], out=out, fmt_a=fa, fmt_b=fb, preset=nfma, fast=fast,
                                 scale_result=sc[2] if out.startswith("float8") else None)
        assert np.array_equal(got.view(truth.dtype), truth), "the two GPU entry points agree with each other but not " \
                                                             "with the oracle"
        assert L.mmb200_scaled_mm_static_status(a.shape[0], b.shape[0], a.shape[1], None) == _lib.OK


def test_static_scratch_entry_point_refuses_what_it_cannot_serve():
    L = _lib.load()
    assert L.mmb200_workspace_bytes(4096, 4096, 4096) > 64 << 20
    dummy = torch.zeros(4096 * 16, dtype=torch.uint8, device=DEV)
    s = torch.ones(2, device=DEV)
    p = dummy.data_ptr()
    common = (p, 4096, 0, p, 4096, 0, p, 4096, 1)
    assert L.mmb200_scaled_mm_static(*common, 4096, 4096, 4096, 32, 1, s.data_ptr(), s.data_ptr() + 4, None, None) \
        == _lib.ERR_TOO_LARGE
    assert L.mmb200_scaled_mm_static(p + 8, 64, 0, p, 64, 0, p, 64, 1, 16, 16, 64, 32, 1, s.data_ptr(), s.data_ptr() + 4,
                                     None, None) == _lib.ERR_UNSUPPORTED          # operand not 16-byte aligned
    assert L.mmb200_scaled_mm_static(p, 72, 0, p, 72, 0, p, 64, 1, 16, 16, 72, 32, 1, s.data_ptr(), s.data_ptr() + 4,
                                     None, None) == _lib.ERR_UNSUPPORTED          # K not a multiple of 16
    torch.cuda.synchronize(DEV)
