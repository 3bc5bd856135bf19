"""Puts the unmodified reference (astding/mmaemu) under baseline/_ref/ so that it can be imported beside this package.

    python baseline/install_reference.py [--reference DIR] [--no-tests]

baseline/_ref/ is never committed; it travels with a checkout to the machine that has the GPU. It is used by
  - tests/test_reference_kernels_gpu.py: the reference's own CUDA kernels (cuda:h4, cuda:h1, cuda:v4, cuda:v1) loaded
    by the reference's stock loader and compared bit for bit with this package on the same device;
  - tests/test_reference_suite_gpu.py: the reference's own GPU test files run with backend "cuda:b200";
  - bench.py: the reference's CPU backend (`--impl reference`, `cpu_baseline`) and its h4 kernel timed as context.

The project builds with hatchling, which is not installed here, so `pip install --target` cannot make the wheel; a wheel
of this project is its `mmaemu/` package directory and nothing else (pyproject.toml, [tool.hatch.build.targets.wheel]),
so the directory is copied as it is, and every copied file is compared with its source byte for byte. The reference's
tests/ directory (test files and their data) and tools/record/ (the input generator its tests import) are copied to
baseline/_ref/tests/ and baseline/_ref/tools/record/ as well, unless --no-tests is given.
"""
from __future__ import annotations

import argparse
import filecmp
import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"


def default_reference() -> Path:
    return Path(os.environ.get("MMAEMU_REFERENCE", str(HERE.parents[1] / "reference")))


def _copy_tree(src: Path, dst: Path) -> int:
    if dst.exists():
        shutil.rmtree(dst)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc", ".pytest_cache"))
    n = 0
    for f in src.rglob("*"):
        if f.is_file() and "__pycache__" not in f.parts and f.suffix != ".pyc" and ".pytest_cache" not in f.parts:
            if not filecmp.cmp(f, dst / f.relative_to(src), shallow=False):
                raise RuntimeError(f"copy of {f} differs from its source")
            n += 1
    return n


def installed() -> bool:
    return (DEST / "mmaemu" / "__init__.py").exists()


def install(reference: Path | None = None, with_tests: bool = True, quiet: bool = False) -> bool:
    """Copy the package (and tests). Returns False, doing nothing, when the reference tree is absent."""
    ref = Path(reference) if reference else default_reference()
    if not (ref / "mmaemu" / "__init__.py").exists():
        return False
    DEST.mkdir(parents=True, exist_ok=True)
    n = _copy_tree(ref / "mmaemu", DEST / "mmaemu")
    if with_tests and (ref / "tests").is_dir():
        n += _copy_tree(ref / "tests", DEST / "tests")
        if (ref / "tools" / "record").is_dir():        # the input generator of the recorded H100 calls (tests import it)
            n += _copy_tree(ref / "tools" / "record", DEST / "tools" / "record")
    if not quiet:
        print(f"installed {n} files of {ref} under {DEST}")
    return True


def add_to_path() -> bool:
    """Make `import mmaemu` find the installed copy. Returns False when nothing is installed."""
    if not installed():
        return False
    if str(DEST) not in sys.path:
        sys.path.insert(0, str(DEST))
    return True


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--reference", default=None)
    ap.add_argument("--no-tests", action="store_true")
    a = ap.parse_args()
    ok = install(a.reference, with_tests=not a.no_tests)
    if not ok:
        sys.exit(f"no reference tree at {a.reference or default_reference()}")
