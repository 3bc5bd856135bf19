"""Pin the C oracle against the reference itself (run in a container that has the reference tree; not at GPU run time).

The reference's own test-suite for the hot path is run with the reference's *compute* swapped for the C oracle, while
the reference keeps doing validation, split-K resolution and test bookkeeping:

  mmaemu.api.execute_plan        -> oracle.accumulate   (plan.py:169-208 + chain.py:286-332 + specials.py:25-80)
  mmaemu.model.epilogue.apply    -> oracle.epilogue     (epilogue.py:65-78)
  mmaemu.model.chain._dot_values -> oracle.dot          (chain.py:107-117, the instruction-level chain)

So every golden vector those tests hold becomes a check of the oracle: the 2,519 RTX 4060 hardware cases of
tests/data/hw_mini, the 124 H100 PCIe live calls of tests/data/h100_mini (sha256 of the hardware output), the 64
recorded epilogue ties and hardware extracts of tests/data/epilogue, the 50,000 MATLAB-toolbox instruction vectors, the
hard-coded hardware bytes in tests/test_api.py, and the unit tests of the plan layouts and reduction orders.

usage:  python oracle/pin_against_reference.py [--reference <checkout of astding/mmaemu>] [pytest args]
Prints how many calls were served by the oracle and how many fell back to the reference's own code (custom presets,
non-finite instruction-level operands), then pytest's summary. Exit code = pytest's.
"""
from __future__ import annotations

import argparse
import os
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

DEFAULT_TESTS = ["test_hw_mini.py", "test_h100_mini.py", "test_epilogue.py", "test_toolbox_vectors.py",
                 "test_plan.py", "test_model_chain.py", "test_specials.py", "test_api.py"]
COUNTS = {"accumulate": 0, "accumulate_fallback": 0, "epilogue": 0, "dot": 0, "dot_fallback": 0}


class OraclePatch:
    """pytest plugin: installs the patches once the reference package is importable."""

    def pytest_configure(self, config):
        import torch
        import mmaemu.api as api
        import mmaemu.backends.reference as ref_backend
        import mmaemu.model.chain as chain
        import mmaemu.model.epilogue as epilogue
        import mmaemu.model.plan as plan
        from mmaemu.model import presets
        from oracle import oracle

        def nfma_of(p):
            """The oracle's preset code: 16 / 32 for the two early-accumulator presets, 288 for the late-accumulator
            b200_mma_sync (32 products, 25 / 23 fraction bits); None (fall back) for anything else."""
            if isinstance(p, str):
                p = presets._lookup(p)[0]
            if p.late_c:
                return 288 if (p.nfma, p.frac, p.frac_out, p.min_exp) == (32, 25, 23, -133) else None
            if p.frac != 13 or p.frac_out != 13 or p.nfma not in (16, 32):
                return None
            return p.nfma

        orig_chain_fn = ref_backend.ReferenceBackend.chain_fn

        def chain_fn(self, req):
            fn = orig_chain_fn(self, req)
            fn.oracle_nfma = nfma_of(req.preset)
            return fn
        ref_backend.ReferenceBackend.chain_fn = chain_fn

        orig_execute = plan.execute_plan

        def execute_plan(pl, a_u8, b_u8, *, fmt_a, fmt_b, chain_fn):
            nf = getattr(chain_fn, "oracle_nfma", None)
            if (nf is None or a_u8.dtype != torch.uint8 or b_u8.dtype != torch.uint8 or a_u8.dim() != 2
                    or b_u8.dim() != 2 or a_u8.shape[1] != b_u8.shape[1] or a_u8.shape[1] != pl.K
                    or a_u8.device.type != "cpu"):
                COUNTS["accumulate_fallback"] += 1
                return orig_execute(pl, a_u8, b_u8, fmt_a=fmt_a, fmt_b=fmt_b, chain_fn=chain_fn)
            COUNTS["accumulate"] += 1
            bits = oracle.accumulate(a_u8.contiguous().numpy(), b_u8.contiguous().numpy(), fmt_a=fmt_a, fmt_b=fmt_b,
                                     preset=nf, fast=pl.fast, S=pl.S, scheme=pl.scheme)
            return torch.from_numpy(bits.view(np.int32).copy()).view(torch.float32)
        plan.execute_plan = execute_plan
        api.execute_plan = execute_plan

        def apply(acc32, scale_a, scale_b, *, out_dtype, scale_result=None):
            if acc32.dtype != torch.float32:
                raise TypeError(f"acc32 must be float32, got {acc32.dtype}")
            COUNTS["epilogue"] += 1
            name = str(out_dtype).replace("torch.", "")
            sr = None if scale_result is None else float(scale_result.to(torch.float32).reshape(()).item())
            bits = oracle.epilogue(acc32.detach().cpu().contiguous().view(torch.int32).numpy().view(np.uint32),
                                   float(scale_a.to(torch.float32).reshape(()).item()),
                                   float(scale_b.to(torch.float32).reshape(()).item()), out=name, scale_result=sr)
            it = {1: (np.uint8, torch.uint8), 2: (np.int16, torch.int16), 4: (np.int32, torch.int32)}[bits.itemsize]
            return torch.from_numpy(bits.view(it[0]).copy()).view(out_dtype).reshape(acc32.shape).to(acc32.device)
        epilogue.apply = apply

        orig_dot_values = chain._dot_values

        def _dot_values(a, b, c, p, fmt):
            nf = nfma_of(p)
            fa, fb = (fmt, fmt) if isinstance(fmt, str) else fmt
            finite = bool(torch.isfinite(a).all()) and bool(torch.isfinite(b).all()) and (
                c is None or bool(torch.isfinite(c).all()))
            if nf is None or not finite or a.device.type != "cpu":
                COUNTS["dot_fallback"] += 1
                return orig_dot_values(a, b, c, p, fmt)
            COUNTS["dot"] += 1
            from mmaemu.formats import DTYPE_OF
            K = a.shape[-1]
            ac = a.to(DTYPE_OF[fa]).view(torch.uint8).reshape(-1, K).contiguous().numpy()
            bc = b.to(DTYPE_OF[fb]).view(torch.uint8).reshape(-1, K).contiguous().numpy()
            cc = None if c is None else c.to(torch.float32).reshape(-1).contiguous().view(torch.int32).numpy().view(
                np.uint32)
            d = oracle.dot(ac, bc, cc, fmt_a=fa, fmt_b=fb, preset=nf)
            return torch.from_numpy(d.view(np.int32).copy()).view(torch.float32).reshape(a.shape[:-1]).double()
        chain._dot_values = _dot_values

    def pytest_terminal_summary(self, terminalreporter):
        terminalreporter.write_line("oracle pin: " + ", ".join(f"{k}={v}" for k, v in COUNTS.items()))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--reference", default=os.environ.get("MMAEMU_REFERENCE", str(Path(__file__).resolve().parents[2] / "reference")))
    ap.add_argument("--tests", nargs="*", default=DEFAULT_TESTS)
    args, rest = ap.parse_known_args(argv)
    ref = Path(args.reference)
    if not (ref / "mmaemu" / "__init__.py").is_file():
        print(f"reference tree not found at {ref}", file=sys.stderr)
        return 2
    sys.path.insert(0, str(ref))
    sys.dont_write_bytecode = True
    os.environ["PYTHONDONTWRITEBYTECODE"] = "1"
    import pytest
    from oracle import oracle
    oracle.build()
    work = tempfile.mkdtemp(prefix="oracle_pin_")
    os.chdir(work)                                   # the reference tree is read-only
    files = [str(ref / "tests" / t) for t in args.tests]
    return int(pytest.main(["-q", "-x", "-p", "no:cacheprovider", "-m", "not gpu and not slow and not truth",
                            f"--rootdir={ref}", "-c", str(ref / "pyproject.toml"), *rest, *files],
                           plugins=[OraclePatch()]))


if __name__ == "__main__":
    sys.exit(main())
