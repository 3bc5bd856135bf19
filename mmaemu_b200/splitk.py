"""Split-K resolution: which (S, reduction scheme) cuBLASLt uses for a GEMM on the profile's emulated platform.

Host logic in front of the kernels; it restates the reference's resolver (astding/mmaemu,
mmaemu/platform/splitk_table.py:341-465) over the same recorded heuristic tables (imported by
mmaemu_b200/data/import_tables.py). Order of resolution:

  1. explicit      splitk is 1, a SplitK or an (S, scheme) tuple (an int > 1 without a scheme is a ValueError);
  2. workspace0    a profile without cuBLASLt workspace never splits;
  3. table         the shape is a row of the profile's table: the recorded numSplitsK and the scheme its customOption
                   maps to;
  4. envelope      S = 1 is inferred for outputs larger than everything that ever split in the setting (RTX 4060:
                   twice the largest split M*N; H100: a bound per setting and K from a K grid), unless strict;
  5. otherwise SplitKUnknownError.
The reference's live cuBLASLt query (between 3 and 4) needs the emulated GPU itself and does not exist on a B200.
Zero-size GEMMs resolve to S = 1. Decisions that were never replayed on hardware warn once per combination
(UnverifiedSplitWarning); envelope inferences of a workspace whose held-out test failed warn
UnvalidatedEnvelopeWarning. `dry=True` (explain) warns every time and does not use up the once.
"""
from __future__ import annotations

import hashlib
import json
import os
import threading
import warnings
from dataclasses import dataclass
from pathlib import Path

import numpy as np

from .errors import SplitKUnknownError, UnvalidatedEnvelopeWarning, UnverifiedSplitWarning
from .numerics import ALL_SCHEMES, SPLIT_SCHEMES
from .platforms import get_profile

DATA = Path(__file__).resolve().parent / "data"
OUT_CODES = {"float32": 0, "bfloat16": 1, "float16": 2, "float8_e4m3fn": 3, "float8_e5m2": 4}
FMT_CODES = {"e4m3": 0, "e5m2": 1}
_FMT_NAMES = {"float8_e4m3fn": "e4m3", "float8_e5m2": "e5m2", "e4m3": "e4m3", "e5m2": "e5m2"}
CONTIG_TILE_K = 128
ENVELOPE_MARGIN = 2          # RTX 4060: S = 1 is inferred only above twice the largest M*N that split
_DIM_LIMIT = 1 << 21


@dataclass(frozen=True)
class SplitK:
    """An explicit split: S partial sums combined with `scheme`."""
    S: int = 1
    scheme: str = "none"

    def __post_init__(self):
        if isinstance(self.S, bool) or not isinstance(self.S, (int, np.integer)) or self.S < 1:
            raise ValueError(f"SplitK.S must be an int >= 1, got {self.S!r}")
        if self.S == 1 and self.scheme != "none":
            raise ValueError(f"S = 1 has no reduction scheme (got {self.scheme!r}); use scheme='none'")
        if self.S > 1 and self.scheme not in ALL_SCHEMES:
            raise ValueError(f"S = {self.S} requires scheme 'serial', 'pairwise' or 'contiguous', got {self.scheme!r}")


@dataclass(frozen=True)
class SplitDecision:
    S: int
    scheme: str
    source: str           # "explicit" | "workspace0" | "table" | "envelope"
    verified: bool
    table_id: str | None
    note: str

    @property
    def splitk(self) -> SplitK:
        return SplitK(self.S, self.scheme)


def _name(dt):
    if dt is None:
        return None
    s = str(dt)
    return s[6:] if s.startswith("torch.") else s


def _fmt(dt, what):
    s = _name(dt)
    if s not in _FMT_NAMES:
        raise TypeError(f"{what} must be float8_e4m3fn or float8_e5m2 (or 'e4m3'/'e5m2'), got {dt!r}")
    return _FMT_NAMES[s]


class SplitTable:
    """One imported heuristic table; rows are found by binary search on (setting, M, N, K)."""

    def __init__(self, table_id: str, data_dir: Path = DATA):
        self.id = table_id
        self.meta = json.loads((data_dir / f"{table_id}.json").read_text())
        raw = (data_dir / f"{table_id}.npz").read_bytes()
        if hashlib.sha256(raw).hexdigest() != self.meta["npz_sha256"]:
            raise RuntimeError(f"{table_id}.npz does not match the sha256 recorded in {table_id}.json")
        import io
        z = np.load(io.BytesIO(raw), allow_pickle=False)
        self.ws_values = [int(w) for w in self.meta["ws"]]
        i64 = np.int64
        setting = ((z["ws"].astype(i64) << 16) | (z["out"].astype(i64) << 8) | (z["fast"].astype(i64) << 4)
                   | (z["fa"].astype(i64) << 2) | z["fb"].astype(i64))
        shape = (z["M"].astype(i64) << 42) | (z["N"].astype(i64) << 21) | z["K"].astype(i64)
        order = np.lexsort((shape, setting))
        self._setting, self._shape = setting[order], shape[order]
        self._splits, self._custom = z["splitK"][order], z["custom"][order]
        self._settings = {(int(s["ws"]), s["out"], bool(s["fast"]), s["fmt_a"], s["fmt_b"]): s
                          for s in self.meta["settings"]}
        self.verified = {(bool(c[0]), int(c[1]), c[2], c[3], c[4]) for c in self.meta["verified_combos"]}
        self._rule = {str(k): v for k, v in self.meta["custom_to_scheme"].items()}
        self._unlisted = self.meta.get("custom_to_scheme_unlisted")
        env = self.meta.get("envelope") or {}
        self.envelope_inference = bool(env.get("inference", True))
        self.envelope_note = env.get("note", "")
        self.envelope_kind = env.get("kind", "max_split_MN")
        if self.envelope_kind == "k_grid":
            self.k_grid = np.asarray(env["K_grid"], dtype=np.int64)
            self.k_min, self.k_max = int(env["K_min"]), int(env["K_max"])
            self.k_bounds = {(int(b["ws"]), b["out"], bool(b["fast"]), b["fmt_a"], b["fmt_b"]): b["B"]
                             for b in env["bounds"]}
            self.k_validation = {int(w): v for w, v in env["validation"].items()}
            self.envelope_eval = env.get("eval", "")
        elif self.envelope_kind != "max_split_MN":
            raise RuntimeError(f"{table_id}.json: unknown envelope kind {self.envelope_kind!r}")
        self.ragged_verified = bool(self.meta.get("ragged_K_verified", False))
        self.workspace0_note = self.meta.get("workspace0_note") or "cuBLASLt never splits without a workspace"

    def scheme_of(self, custom):
        """(scheme, caveat) of a split row's customOption."""
        c = str(int(custom))
        if c in self._rule:
            return self._rule[c], None
        if self._unlisted is None:
            return "serial", None
        return self._unlisted, (f"customOption {c} was never recorded on a split call (recorded: "
                                f"{', '.join(sorted(self._rule))})")

    def lookup(self, M, N, K, fmt_a, fmt_b, out, fast, ws):
        """{'splitK', 'custom'} of the table row, or None."""
        if ws not in self.ws_values or out not in OUT_CODES or max(M, N, K) >= _DIM_LIMIT or min(M, N, K) < 0:
            return None
        s = ((self.ws_values.index(ws) << 16) | (OUT_CODES[out] << 8) | (int(bool(fast)) << 4)
             | (FMT_CODES[fmt_a] << 2) | FMT_CODES[fmt_b])
        lo, hi = np.searchsorted(self._setting, s, "left"), np.searchsorted(self._setting, s, "right")
        if lo == hi:
            return None
        key = (int(M) << 42) | (int(N) << 21) | int(K)
        i = lo + int(np.searchsorted(self._shape[lo:hi], key))
        if i >= hi or int(self._shape[i]) != key:
            return None
        return {"splitK": int(self._splits[i]), "custom": int(self._custom[i])}

    def k_bound(self, K, ws, out, fast, fmt_a, fmt_b):
        """(bound on M*N above which S = 1 is inferred, how) or (None, why not), for a 'k_grid' envelope."""
        if not self.k_min <= K <= self.k_max:
            return None, f"K = {K} is outside the envelope's K range {self.k_min:,}..{self.k_max:,}"
        b = self.k_bounds.get((int(ws), out, bool(fast), fmt_a, fmt_b))
        if b is None:
            return None, f"the envelope has no bound at workspace {ws} B for this setting"
        i = int(np.searchsorted(self.k_grid, K, side="left"))
        if b[i] is None:
            return None, f"the envelope infers nothing from grid K = {int(self.k_grid[i]):,} on"
        return int(b[i]), f"bound {int(b[i]):,} at grid K = {int(self.k_grid[i]):,} (the smallest grid K >= {K})"

    def envelope(self, ws, out, fast, fmt_a, fmt_b):
        """(per-setting envelope, how it was obtained) or (None, why) for a 'max_split_MN' envelope. A setting absent
        from the table uses the union over output dtypes of the same (ws, fast, format pair)."""
        st = self._settings.get((int(ws), out, bool(fast), fmt_a, fmt_b))
        if st is not None:
            return st, "setting"
        same = [v for (w, o, f, a, b), v in self._settings.items() if (w, f, a, b) == (int(ws), bool(fast), fmt_a, fmt_b)]
        if not same:
            return None, f"no table rows for ws={ws}, fast={fast}, {fmt_a}x{fmt_b}"
        sp = [v for v in same if v["split_rows"]]
        env = dict(rows=sum(v["rows"] for v in same), split_rows=sum(v["split_rows"] for v in same),
                   max_split_MN=max((v["max_split_MN"] for v in sp), default=None),
                   min_split_K=min((v["min_split_K"] for v in sp), default=None))
        return env, f"union over output dtypes {sorted(v['out'] for v in same)} (setting {out} absent)"


_TABLES: dict = {}
_LOCK = threading.Lock()
_WARNED: set = set()


def load_table(table_id: str) -> SplitTable:
    with _LOCK:
        t = _TABLES.get(table_id)
        if t is None:
            t = _TABLES[table_id] = SplitTable(table_id)
        return t


def _reset_warnings_for_tests() -> None:
    with _LOCK:
        _WARNED.clear()


def _scheme_hint(p, S="S") -> str:
    schemes = SPLIT_SCHEMES.get(p.preset) or ALL_SCHEMES
    return f"({S}, " + "|".join(repr(x) for x in schemes) + ")"


def _layout_caveat(K, S, scheme, table):
    """Why a contiguous split lies outside the replayed calls although its combination was replayed."""
    if scheme != "contiguous" or S <= 1:
        return None
    T = -(-K // CONTIG_TILE_K)
    if K % CONTIG_TILE_K and not (table is not None and table.ragged_verified):
        return f"K = {K} is not a multiple of {CONTIG_TILE_K} (no replayed split call has a ragged last k-tile)"
    if (S - 1) * -(-T // S) >= T:
        return f"S = {S} leaves a split without k-tiles (K = {K}, {T} k-tiles; never recorded)"
    return None


def _once(key, dry) -> bool:
    """True if the warning keyed by `key` should be emitted now."""
    if dry:
        return True
    with _LOCK:
        if key in _WARNED:
            return False
        _WARNED.add(key)
        return True


def _warn_split(p, fast, S, scheme, out, pair, verified, source, dry, caveat):
    experimental = S > 1 and p.splitk_maturity == "experimental"
    if verified and not experimental:
        return
    if not _once((p.name, bool(fast), S, scheme, out, pair) + ((caveat,) if caveat else ()), dry):
        return
    if not verified:
        why = caveat or "this (fast, S, scheme, out, format pair) combination was never replayed on hardware"
    else:
        why = f"split-K decisions of profile {p.name} are experimental"
    warnings.warn(f"mmaemu split-K S={S} scheme={scheme} ({'fast' if fast else 'slow'} accumulation, out {out}, "
                  f"{pair}, source {source}, profile {p.name}): {why}", UnverifiedSplitWarning, stacklevel=4)


def _warn_envelope(p, table, ws, out, fast, pair, val, dry):
    if not _once((p.name, "envelope", ws, out, bool(fast), pair), dry):
        return
    why = ("this workspace's envelope has no held-out test" if val is None else
           f"this workspace's envelope did not pass its held-out test ({val['split_above_bound']} of "
           f"{val['tested']:,} held-out shapes above the bound split on the {p.gpu_name}; {table.envelope_eval})")
    warnings.warn(f"mmaemu split-K S=1 inferred by the envelope of table {table.id} (workspace {ws} B, "
                  f"{'fast' if fast else 'slow'} accumulation, out {out}, {pair}, profile {p.name}): {why}, so the GPU "
                  f"may split this shape. Pass splitk explicitly, or set MMAEMU_SPLITK_STRICT=1 to refuse the inference",
                  UnvalidatedEnvelopeWarning, stacklevel=4)


def _explicit(splitk, p):
    if isinstance(splitk, SplitK):
        return splitk
    if all(hasattr(splitk, f) for f in ("S", "scheme")) and not isinstance(splitk, tuple):
        return SplitK(int(splitk.S), splitk.scheme)          # a SplitK of the reference package
    if isinstance(splitk, (int, np.integer)) and not isinstance(splitk, bool):
        if splitk > 1:
            raise ValueError(f"splitk={splitk} needs a reduction scheme: pass splitk={_scheme_hint(p, splitk)}")
        return SplitK(int(splitk), "none")
    if isinstance(splitk, tuple) and len(splitk) == 2:
        return SplitK(splitk[0], splitk[1])
    raise TypeError(f"splitk must be 'auto', 1, a SplitK or an (S, scheme) tuple, got {splitk!r}")


def resolve_splitk(M, N, K, *, a_dtype, b_dtype, out_dtype, use_fast_accum, profile=None, splitk="auto",
                   layout_std=True, strict=None, dry=False) -> SplitDecision:
    """The split-K decision for torch._scaled_mm(a[M, K], b[K, N]) on the profile's platform (module docstring).
    out_dtype None means a_dtype, as torch."""
    p = get_profile(profile)
    fa, fb = _fmt(a_dtype, "a_dtype"), _fmt(b_dtype, "b_dtype")
    out = _name(out_dtype) or _name(a_dtype)
    out = {"e4m3": "float8_e4m3fn", "e5m2": "float8_e5m2"}.get(out, out)
    if out not in OUT_CODES:
        raise TypeError(f"out_dtype must be one of {sorted(OUT_CODES)}, got {out_dtype!r}")
    fast, pair = bool(use_fast_accum), f"{fa}x{fb}"
    M, N, K = int(M), int(N), int(K)
    if strict is None:
        strict = os.environ.get("MMAEMU_SPLITK_STRICT") == "1"
    table = load_table(p.splitk_table) if p.splitk_table else None
    verified = table.verified if table is not None else set()

    def decided(S, custom, source, prefix):
        scheme, cav = ("none", None) if S <= 1 else table.scheme_of(custom)
        cav = cav or _layout_caveat(K, S, scheme, table)
        ok = S == 1 or ((fast, S, scheme, out, pair) in verified and cav is None)
        _warn_split(p, fast, S, scheme, out, pair, ok, source, dry, cav)
        return SplitDecision(S, scheme, source, ok, table.id if source == "table" else None,
                             prefix + (f"; {cav}" if cav else ""))

    if not (isinstance(splitk, str) and splitk == "auto"):                       # 1. explicit
        sk = _explicit(splitk, p)
        cav = _layout_caveat(K, sk.S, sk.scheme, table)
        ok = sk.S == 1 or ((fast, sk.S, sk.scheme, out, pair) in verified and cav is None)
        _warn_split(p, fast, sk.S, sk.scheme, out, pair, ok, "explicit", dry, cav)
        return SplitDecision(int(sk.S), sk.scheme, "explicit", ok, None, "given by the caller" + (f"; {cav}" if cav else ""))
    if p.workspace_bytes == 0:                                                   # 2. no workspace
        return SplitDecision(1, "none", "workspace0", True, p.splitk_table,
                             table.workspace0_note if table is not None else "cuBLASLt never splits without a workspace")
    ways_out = (f"Ways out: pass splitk=1 if the call is known to be unsplit; splitk={_scheme_hint(p)} if the split is "
                f"known")
    if p.workspace_bytes is None or table is None:
        raise SplitKUnknownError(f"profile {p.name!r} has no reference platform and no split-K table, so "
                                 f"splitk='auto' cannot be resolved for M={M} N={N} K={K}. {ways_out}")
    ws = p.workspace_bytes
    if min(M, N, K) == 0:
        return SplitDecision(1, "none", "envelope", True, p.splitk_table, "zero-size GEMM: nothing is accumulated")
    if layout_std:                                                               # 3. table
        row = table.lookup(M, N, K, fa, fb, out, fast, ws)
        if row is not None:
            return decided(row["splitK"], row["custom"], "table",
                           f"table row: numSplitsK {row['splitK']}, customOption {row['custom']}")
    where = f"M={M} N={N} K={K} on profile {p.name!r}"
    setting = f"(ws={ws} B, out={out}, {'fast' if fast else 'slow'} accumulation, {pair})"
    if not table.envelope_inference:                                             # 4. envelope
        why = "the shape is not in the table" if layout_std else "the layout is not torch's standard one"
        raise SplitKUnknownError(f"split-K decision unknown for {where}: {why} and table {table.id} infers nothing "
                                 f"outside its rows ({table.envelope_note}). {ways_out}")
    if table.envelope_kind == "k_grid":
        B, how = table.k_bound(K, ws, out, fast, fa, fb)
        val = table.k_validation.get(ws)
        if B is not None and M * N > B and not strict:
            ok = val is not None and val["status"] == "validated"
            if not ok:
                _warn_envelope(p, table, ws, out, fast, pair, val, dry)
            state = ("unvalidated (no held-out test)" if val is None else
                     f"{val['status']} on held-out shapes ({val['tested']:,} above the bound, "
                     f"{val['split_above_bound']} split; {table.envelope_eval})")
            return SplitDecision(1, "none", "envelope", ok, table.id,
                                 f"inference: M*N = {M * N} is above the envelope {how} of setting {setting}; "
                                 f"envelope {state}")
        if B is None:
            reason = f"the shape is not in the table and {how}"
        elif M * N > B:
            reason = "strict mode (MMAEMU_SPLITK_STRICT=1 or strict=True)"
        else:
            reason = f"the shape is not in the table and M*N = {M * N} is not above the envelope {how} of setting {setting}"
        raise SplitKUnknownError(f"split-K decision unknown for {where}: {reason}. {ways_out}; or run the call on the "
                                 f"profile's {p.gpu_name}")
    env, how = table.envelope(ws, out, fast, fa, fb)
    if env is None:
        outside, env_s = False, f"no envelope for setting {setting}: {how}"
    elif not env["split_rows"]:
        outside, env_s = True, f"split envelope of setting {setting} [{how}]: none of its {env['rows']} rows split"
    else:
        mx = env["max_split_MN"]
        outside = M * N > ENVELOPE_MARGIN * mx
        env_s = (f"inference bound {ENVELOPE_MARGIN} x {mx} = {ENVELOPE_MARGIN * mx} of setting {setting} [{how}] "
                 f"(largest split M*N {mx}; {env['split_rows']} of {env['rows']} rows split)")
    if outside and not strict:
        return SplitDecision(1, "none", "envelope", True, table.id, f"inference: M*N = {M * N} is above the {env_s}")
    if env is None:
        reason = "the table has no rows for this setting"
    elif outside:
        reason = "strict mode (MMAEMU_SPLITK_STRICT=1 or strict=True)"
    else:
        reason = f"the shape is not in the table and M*N = {M * N} is not above the inference bound"
    raise SplitKUnknownError(f"split-K decision unknown for {where}: {reason}; {env_s}. {ways_out}")
