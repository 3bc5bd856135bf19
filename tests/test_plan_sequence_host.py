"""The k-tile sequence that drives split plans on the staged kernels (mmaemu_b200/csrc/plan.cuh, plan_sequence),
compiled for the host and checked without a GPU.

The sequence is consumed exactly as the kernels consume it -- block steps over the listed 32-element k-tiles, a chain
end where the entry says so, the split's partial entering the reduction in its role -- with the oracle's single-chain
primitive (oracle.dot) standing in for the block steps; the result must equal the oracle's own execution of the plan
(oracle.accumulate), bit for bit, for every scheme, split count, accumulation mode and ragged K."""
import ctypes
import subprocess
from pathlib import Path

import numpy as np
import pytest

import datagen
from oracle import oracle

HERE = Path(__file__).resolve().parent
SRC = HERE / "host" / "plan_host.cpp"
LIB = HERE / "host" / "_build" / "libplan_host.so"
SCHEME = {"none": 0, "serial": 1, "pairwise": 2, "contiguous": 3}
TILE_MASK, CHAIN_END, SPLIT_END, EMPTY, ROLE_SHIFT = 0xFFFFF, 1 << 20, 1 << 21, 1 << 22, 24


@pytest.fixture(scope="module")
def lib():
    hdr = HERE.parent / "mmaemu_b200" / "csrc" / "plan.cuh"
    if not LIB.exists() or LIB.stat().st_mtime < max(SRC.stat().st_mtime, hdr.stat().st_mtime):
        LIB.parent.mkdir(exist_ok=True)
        subprocess.run(["g++", "-O1", "-fPIC", "-shared", "-std=c++17", str(SRC), "-o", str(LIB)], check=True)
    L = ctypes.CDLL(str(LIB))
    L.plan_sequence_host.argtypes = [ctypes.c_int] * 4 + [ctypes.c_void_p, ctypes.c_int]
    L.plan_sequence_host.restype = ctypes.c_int
    return L


def sequence(L, K, fast, S, scheme):
    buf = np.zeros(K // 32 + S + 16, np.uint32)
    n = L.plan_sequence_host(K, int(fast), S, SCHEME[scheme], buf.ctypes.data, buf.size)
    assert n > 0
    return buf[:n]


def walk(seq, a, b, nfma, fast):
    """Diagonal outputs (row i of a with row i of b) computed by consuming the sequence the way the kernels do."""
    rows, K = a.shape
    f32 = np.float32
    tot = np.zeros(rows, f32)
    slot = np.zeros(rows, f32)
    part = np.zeros(rows, f32)
    cols = []                                   # k indices of the chain in progress

    def chain():
        nonlocal cols
        if not cols:
            return np.zeros(rows, f32)
        idx = np.concatenate(cols)
        cols = []
        return oracle.dot(a[:, idx], b[:, idx], None, preset=nfma).view(f32)
    for e in seq:
        e = int(e)
        if not e & EMPTY:
            k0 = (e & TILE_MASK) * 32
            cols.append(np.arange(k0, min(k0 + 32, K)))
        if e & CHAIN_END:
            assert not fast
            part = part + chain()
        if e & SPLIT_END:
            pv = chain() if fast else part
            assert fast or not cols             # slow accumulation: no tiles pending at a split end
            role = (e >> ROLE_SHIFT) & 7
            if role == 0:
                tot = pv
            elif role == 1:
                slot = pv
            elif role == 2:
                tot = tot + (slot + pv)
            else:
                tot = tot + pv
            part = np.zeros(rows, f32)
    assert not cols
    return tot.view(np.uint32)


CASES = [(S, scheme) for scheme in ("serial", "pairwise") for S in (2, 3, 5, 8, 12, 29)] + \
        [(S, "contiguous") for S in (2, 3, 4, 6, 7, 24)]


@pytest.mark.parametrize("fast", (True, False), ids=("fast", "slow"))
@pytest.mark.parametrize("S,scheme", CASES, ids=lambda v: str(v))
def test_sequence_reproduces_the_plan(lib, S, scheme, fast):
    nfma = 32 if scheme == "contiguous" else 16
    rng = np.random.default_rng(S * 7 + len(scheme))
    for K in (64, 208, 1024, 1936, 4112):       # including K below one tile per split (empty splits) and ragged tiles
        a = datagen.codes(rng, 24, K, "e4m3", "gauss40", 0)
        b = datagen.codes(rng, 24, K, "e4m3", "block_exponents", 1)
        seq = sequence(lib, K, fast, S, scheme)
        tiles = [int(e) & TILE_MASK for e in seq if not int(e) & EMPTY]
        assert sorted(tiles) == list(range((K + 31) // 32))          # every k-tile exactly once
        assert sum(1 for e in seq if int(e) & SPLIT_END) == S
        got = walk(seq, a, b, nfma, fast)
        want = np.array([oracle.accumulate(a[i:i + 1], b[i:i + 1], preset=nfma, fast=fast, S=S, scheme=scheme)[0, 0]
                         for i in range(a.shape[0])], dtype=np.uint32)
        assert np.array_equal(got, want), (K, S, scheme, fast)


@pytest.mark.parametrize("fast", (True, False), ids=("fast", "slow"))
@pytest.mark.parametrize("S,scheme", [(1, "none")] + CASES, ids=lambda v: str(v))
def test_k_slices_are_whole_chains(lib, S, scheme, fast):
    """The cut of the sequence into K slices: contiguous, covering, every slice with its share of whole chains."""
    lib.plan_slices_host.argtypes = [ctypes.c_int] * 5 + [ctypes.c_void_p] * 2
    lib.plan_slices_host.restype = ctypes.c_int
    for K in (208, 1024, 4112, 32768):
        seq = sequence(lib, K, fast, S, scheme)
        slow = not fast
        emits = [bool(int(e) & CHAIN_END) if slow else bool(int(e) & SPLIT_END and not int(e) & EMPTY) for e in seq]
        chains = sum(emits)
        for slices in sorted({1, 2, 3, 9, 32, chains} & set(range(1, chains + 1))):
            start = np.full(slices + 1, -1, np.int32)
            base = np.full(slices + 1, -1, np.int32)
            assert lib.plan_slices_host(K, int(fast), S, SCHEME[scheme], slices, start.ctypes.data, base.ctypes.data) == chains
            assert start[0] == 0 and start[-1] == len(seq) and base[0] == 0 and base[-1] == chains
            assert (np.diff(start) > 0).all()
            per = np.diff(base)
            assert per.min() >= 1 and per.max() - per.min() <= 1
            for y in range(slices):
                assert sum(emits[start[y]:start[y + 1]]) == per[y]
                if y + 1 < slices:
                    assert emits[start[y + 1] - 1]                    # a slice ends right after a chain's last entry


@pytest.mark.parametrize("fast", (True, False), ids=("fast", "slow"))
def test_workers_write_the_same_sequence(lib, fast):
    """The device kernel fills the sequence with 256 threads; any number of workers must give the serial result."""
    lib.plan_sequence_lanes_host.argtypes = [ctypes.c_int] * 4 + [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
    lib.plan_sequence_lanes_host.restype = ctypes.c_int
    for S, scheme in [(1, "none")] + CASES:
        for K in (64, 208, 1936, 4112, 65552):
            want = sequence(lib, K, fast, S, scheme)
            for lanes in (3, 256):
                buf = np.full(want.size + 4, 0xFFFFFFFF, np.uint32)
                n = lib.plan_sequence_lanes_host(K, int(fast), S, SCHEME[scheme], buf.ctypes.data, buf.size, lanes)
                assert n == want.size and np.array_equal(buf[:n], want) and (buf[n:] == 0xFFFFFFFF).all()


def test_capacity_is_reported(lib):
    buf = np.zeros(4, np.uint32)
    assert lib.plan_sequence_host(4096, 1, 3, SCHEME["contiguous"], buf.ctypes.data, 4) == -128
