"""Converts the reference's recorded cuBLASLt split-K heuristic tables into this package's data files.

The tables are measurements (which numSplitsK / customOption cuBLASLt 12.8.3.14 picked for a shape on the RTX 4060 and
on the H100 PCIe); they cannot be re-derived, so they are imported from a checkout of astding/mmaemu
(mmaemu/platform/data, written there by tools/export_splitk_table.py). Only what split resolution needs is kept: the
key columns, numSplitsK and customOption, the per-setting envelopes, the scheme rule and the verified combinations.

    python mmaemu_b200/data/import_tables.py --reference /path/to/mmaemu

writes <table_id>.npz and <table_id>.json next to this file.
"""
from __future__ import annotations

import argparse
import hashlib
import io
import json
import os
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
TABLES = ("heur_rtx4060_lt12.8.3.14", "heur_h100pcie_lt12.8.3.14")
KEEP = ("M", "N", "K", "fa", "fb", "out", "fast", "ws", "splitK", "custom")


def convert(src: Path, table_id: str) -> None:
    meta = json.loads((src / f"{table_id}.json").read_text())
    raw = (src / f"{table_id}.npz").read_bytes()
    if hashlib.sha256(raw).hexdigest() != meta["npz_sha256"]:
        raise RuntimeError(f"{table_id}.npz does not match the sha256 recorded in its json")
    z = np.load(io.BytesIO(raw), allow_pickle=False)
    cols = {k: z[k] for k in KEEP}
    buf = io.BytesIO()
    np.savez_compressed(buf, **cols)
    (HERE / f"{table_id}.npz").write_bytes(buf.getvalue())
    vc = json.loads((src / meta.get("verified_combos", "verified_split_combos.json")).read_text())
    out = {
        "format": "mmaemu-b200-splitk-table/1",
        "table_id": table_id,
        "source_npz_sha256": meta["npz_sha256"],
        "npz_sha256": hashlib.sha256(buf.getvalue()).hexdigest(),
        "rows": int(len(cols["M"])),
        "profile_device": meta.get("profile_device"),
        "ws": list(meta["codes"]["ws"]),
        "custom_to_scheme": meta["codes"]["custom -> scheme"],
        "custom_to_scheme_unlisted": meta["codes"].get("custom -> scheme, unlisted"),
        "settings": meta["settings"],
        "envelope": meta.get("envelope", {}),
        "ragged_K_verified": bool(meta.get("split_layouts", {}).get("ragged_K", {}).get("verified", False)),
        "workspace0_note": meta.get("workspace0_note"),
        "verified_combos": sorted([bool(c["fast"]), int(c["S"]), c["scheme"], c["out"], c["fmt_pair"]]
                                  for c in vc["combos"] if c["verified"]),
    }
    (HERE / f"{table_id}.json").write_text(json.dumps(out, indent=0, sort_keys=True) + "\n")
    print(table_id, out["rows"], "rows ->", len(buf.getvalue()), "bytes")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("MMAEMU_REFERENCE", str(Path(__file__).resolve().parents[3] / "reference")))
    a = ap.parse_args()
    for t in TABLES:
        convert(Path(a.reference) / "mmaemu" / "platform" / "data", t)
