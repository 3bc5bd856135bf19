"""Regenerates the operand bytes of the H100 PCIe live calls in tests/golden/h100_mini.json (numpy only).

The recorded calls identify their inputs by (data kind, seed, shape, formats); the bytes come from an integer hash, so
they can be rebuilt anywhere. This restates the reference's generator (astding/mmaemu, tools/record/live.py:39-166:
_h32, _key, _u32, _randn_table, make_codes, make_inputs); tests/golden/make_golden.py checks it byte for byte against
that generator before the fixture is written.
"""
from __future__ import annotations

import math

import numpy as np

M32 = np.uint64(0xFFFFFFFF)
C1, C2, C3, C4 = (np.uint64(v) for v in (0x7FEB352D, 0x2C1B3C6D, 0x297A2D39, 0x632BE5AB))
FP8_MAX = {"e4m3": 448.0, "e5m2": 57344.0}


def _mix(x):
    """lowbias32-style 32-bit mix on uint64 arrays holding values < 2^32."""
    x = x ^ (x >> np.uint64(16))
    x = (x * C1) & M32
    x = x ^ (x >> np.uint64(15))
    x = (x * C2) & M32
    return x ^ (x >> np.uint64(16))


def _key(seed: int, salt: int, stream: int) -> np.uint64:
    x = (seed * 0x01000193 + salt * 0x9E37 + stream * 0x3C6EF + 0x3C6EF372) & 0xFFFFFFFF
    for _ in range(2):
        x ^= x >> 16
        x = (x * 0x7FEB352D) & 0xFFFFFFFF
        x ^= x >> 15
        x = (x * 0x2C1B3C6D) & 0xFFFFFFFF
        x ^= x >> 16
    return np.uint64(x)


def _uniform32(seed, salt, stream, rows, cols):
    """uniform 32-bit values [len(rows), len(cols)] (as uint64) from (seed, salt, stream, row, col)."""
    r = _mix((rows ^ _key(seed, salt, stream)) & M32)
    return _mix((r[:, None] + cols[None, :] * C3 + np.uint64(stream) * C4) & M32)


def fp8_value(code: int, fmt: str) -> float:
    """Value of a finite FP8 code."""
    mb, bias = (3, 7) if fmt == "e4m3" else (2, 15)
    e, m = (code & 0x7F) >> mb, code & ((1 << mb) - 1)
    v = (m / (1 << mb)) * 2.0 ** (1 - bias) if e == 0 else (1 + m / (1 << mb)) * 2.0 ** (e - bias)
    return -v if code & 0x80 else v


_TABLES: dict = {}


def _normal_table(fmt: str, scale: float = 40.0):
    """(thresholds uint64 [n], codes uint8 [n + 1]): code = codes[searchsorted(thresholds, u, 'right')] samples the
    distribution of RNE_fp8(clamp(scale * N(0, 1))) from a uniform 32-bit u."""
    if (fmt, scale) not in _TABLES:
        finite = [c for c in range(128) if (c != 0x7F if fmt == "e4m3" else (c & 0x7C) != 0x7C)]
        pos = sorted((fp8_value(c, fmt), c) for c in finite if c != 0)
        ladder = [(-v, c | 0x80) for v, c in reversed(pos)] + [(-0.0, 0x80), (0.0, 0x00)] + pos
        mx = FP8_MAX[fmt]

        def phi(x):
            return 0.5 * (1.0 + math.erf(x / (scale * math.sqrt(2.0))))
        thr = []
        for (a, _), (b, _) in zip(ladder[:-1], ladder[1:]):
            x = 0.0 if (a == 0.0 and b == 0.0) else (a + b) / 2
            cdf = phi(x) if abs(x) < mx else (0.0 if x < 0 else 1.0)
            thr.append(min(0xFFFFFFFF, int(cdf * 2.0 ** 32)))
        _TABLES[(fmt, scale)] = (np.array(thr, dtype=np.uint64), np.array([c for _, c in ladder], dtype=np.uint8))
    return _TABLES[(fmt, scale)]


def _assemble(fmt, sgn, e, m):
    """Code from sign, unbiased exponent (normal range) and a 2-bit mantissa index (1, 1.25, 1.5, 1.75)."""
    if fmt == "e4m3":
        return ((sgn << 7) | ((e + 7) << 3) | (m << 1)).astype(np.uint8)
    return ((sgn << 7) | ((e + 15) << 2) | m).astype(np.uint8)


def make_codes(kind: str, seed: int, rows, K: int, fmt: str, salt: int, S=None) -> np.ndarray:
    """uint8 codes [len(rows), K] of the given row indices for a data kind ('randn40', 'adv', 'adv_split')."""
    rows = np.asarray(list(rows), dtype=np.uint64)
    cols = np.arange(K, dtype=np.uint64)
    if kind == "randn40":
        thr, codes = _normal_table(fmt)
        u = _uniform32(seed, salt, 0, rows, cols)
        return codes[np.searchsorted(thr, u, side="right")]
    if kind == "adv":
        T = -(-K // 64)
        e = (_uniform32(seed, salt, 1, rows, np.arange(T, dtype=np.uint64)) % np.uint64(12)).astype(np.int64) - 6
        e = np.repeat(e, 64, axis=1)[:, :K]
        u = _uniform32(seed, salt, 2, rows, cols).astype(np.int64)
        return _assemble(fmt, (u >> 31) & 1, e, u & 3)
    if kind == "adv_split":
        if not S or S < 2:
            raise ValueError("adv_split needs S >= 2")
        T = -(-K // 64)
        c = np.arange(K, dtype=np.int64)
        t, o = c // 64, c % 64
        sp = t % S

        def full(tt):
            return (tt >= 0) & (tt < T) & ((tt + 1) * 64 <= K)
        q = len(range(S - 1, T, S))
        nm = max(1, q // 2)
        j = t // S
        mir = (sp == S - 1) & full(t) & full(t - (S - 1)) & (j < nm)
        src = (sp == 0) & full(t) & full(t + (S - 1)) & (j < nm)
        hc = np.where(mir, (t - (S - 1)) * 64 + o, c).astype(np.uint64)
        big = (mir | src)[None, :]
        ue = _uniform32(seed, salt, 3, rows, hc).astype(np.int64)
        u = _uniform32(seed, salt, 4, rows, hc).astype(np.int64)
        e = np.where(big, 2 + ue % 3, -6 + ue % 4)
        sgn = (u >> 31) & 1
        if salt == 1:
            sgn = np.where(mir[None, :], 1 - sgn, sgn)
        return _assemble(fmt, sgn, e, u & 3)
    raise ValueError(kind)


def make_inputs(job: dict):
    """(a [M, K], b [N, K]) uint8 code arrays of a recorded job."""
    d = job["data"]
    a = make_codes(d["kind"], d["seed"], range(job["M"]), job["K"], job["fa"], 1, d.get("S"))
    b = make_codes(d["kind"], d["seed"], range(job["N"]), job["K"], job["fb"], 2, d.get("S"))
    return a, b


# ---------------------------------------------------------------------------------------------------------------
# The same generator on torch tensors (any device), for replaying the full recordings on a GPU: all values stay below
# 2^63, so int64 arithmetic reproduces the uint64 arithmetic above. Checked against make_codes in
# tests/test_oracle_golden.py.
def _mix_t(x):
    x = x ^ (x >> 16)
    x = (x * 0x7FEB352D) & 0xFFFFFFFF
    x = x ^ (x >> 15)
    x = (x * 0x2C1B3C6D) & 0xFFFFFFFF
    return x ^ (x >> 16)


def _uniform32_t(seed, salt, stream, rows, cols):
    r = _mix_t((rows ^ int(_key(seed, salt, stream))) & 0xFFFFFFFF)
    return _mix_t((r[:, None] + cols[None, :] * 0x297A2D39 + stream * 0x632BE5AB) & 0xFFFFFFFF)


def make_codes_torch(kind: str, seed: int, row0: int, row1: int, K: int, fmt: str, salt: int, S=None, device="cpu"):
    """uint8 codes [row1 - row0, K] of rows row0..row1-1, as a torch tensor on `device`."""
    import torch
    rows = torch.arange(row0, row1, dtype=torch.int64, device=device)
    cols = torch.arange(K, dtype=torch.int64, device=device)

    def assemble(sgn, e, m):
        if fmt == "e4m3":
            return ((sgn << 7) | ((e + 7) << 3) | (m << 1)).to(torch.uint8)
        return ((sgn << 7) | ((e + 15) << 2) | m).to(torch.uint8)
    if kind == "randn40":
        thr, codes = _normal_table(fmt)
        thr_t = torch.from_numpy(thr.astype(np.int64)).to(device)
        codes_t = torch.from_numpy(codes).to(device)
        u = _uniform32_t(seed, salt, 0, rows, cols)
        return codes_t[torch.searchsorted(thr_t, u, right=True)]
    if kind == "adv":
        T = -(-K // 64)
        e = _uniform32_t(seed, salt, 1, rows, torch.arange(T, dtype=torch.int64, device=device)) % 12 - 6
        e = e.repeat_interleave(64, dim=1)[:, :K]
        u = _uniform32_t(seed, salt, 2, rows, cols)
        return assemble((u >> 31) & 1, e, u & 3)
    if kind == "adv_split":
        if not S or S < 2:
            raise ValueError("adv_split needs S >= 2")
        T = -(-K // 64)
        t, o = cols // 64, cols % 64
        sp = t % S

        def full(tt):
            return (tt >= 0) & (tt < T) & ((tt + 1) * 64 <= K)
        q = len(range(S - 1, T, S))
        nm = max(1, q // 2)
        j = t // S
        mir = (sp == S - 1) & full(t) & full(t - (S - 1)) & (j < nm)
        src = (sp == 0) & full(t) & full(t + (S - 1)) & (j < nm)
        hc = torch.where(mir, (t - (S - 1)) * 64 + o, cols)
        big = (mir | src)[None, :]
        ue = _uniform32_t(seed, salt, 3, rows, hc)
        u = _uniform32_t(seed, salt, 4, rows, hc)
        e = torch.where(big, 2 + ue % 3, -6 + ue % 4)
        sgn = (u >> 31) & 1
        if salt == 1:
            sgn = torch.where(mir[None, :], 1 - sgn, sgn)
        return assemble(sgn, e, u & 3)
    raise ValueError(kind)


def make_inputs_torch(job: dict, device="cpu", chunk_elements: int = 1 << 24):
    """(a [M, K], b [N, K]) uint8 code tensors of a recorded job on `device`, generated in row chunks."""
    import torch
    d = job["data"]
    out = []
    for n_rows, fmt, salt in ((job["M"], job["fa"], 1), (job["N"], job["fb"], 2)):
        x = torch.empty((n_rows, job["K"]), dtype=torch.uint8, device=device)
        step = max(1, chunk_elements // max(1, job["K"]))
        for r0 in range(0, n_rows, step):
            r1 = min(n_rows, r0 + step)
            x[r0:r1] = make_codes_torch(d["kind"], d["seed"], r0, r1, job["K"], fmt, salt, d.get("S"), device)
        out.append(x)
    return out[0], out[1]
