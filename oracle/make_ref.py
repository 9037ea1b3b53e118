"""Recipe for ``oracle/_ref``: an unmodified copy of the reference package (TEST / BENCH INFRASTRUCTURE ONLY).

    python oracle/make_ref.py [--reference <checkout of openvinotoolkit/nncf>]

The reference is pure Python, so "building" it means copying ``<checkout>/src/nncf`` to
``oracle/_ref/nncf`` byte for byte (``__pycache__`` left out).  ``oracle/_ref/`` is git-ignored: the
copy never enters the history, but it travels with the working tree to machines that have no
checkout of the reference, where the benchmark's ``--impl reference`` arm and the boundary test
import it (``oracle.ref_loader``).  Nothing in the product package imports it.

The checkout is found from ``--reference``, else the environment variable ``NNCF_REFERENCE``,
else the sibling directory ``reference`` next to this repository.  When no checkout exists the
script leaves an existing copy alone and reports that nothing was done.
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


def find_checkout(explicit: str | None = None) -> Path | None:
    cands = [explicit, os.environ.get("NNCF_REFERENCE"), str(HERE.parent.parent / "reference")]
    for c in cands:
        if c and (Path(c) / "src" / "nncf" / "__init__.py").exists():
            return Path(c)
    return None


def _same_tree(a: Path, b: Path) -> bool:
    cmp = filecmp.dircmp(a, b, ignore=["__pycache__"])
    if cmp.left_only or cmp.right_only or cmp.funny_files:
        return False
    _, mismatch, errors = filecmp.cmpfiles(a, b, cmp.common_files, shallow=False)
    if mismatch or errors:
        return False
    return all(_same_tree(a / d, b / d) for d in cmp.common_dirs)


def make_ref(reference: str | None = None, verbose: bool = True) -> Path | None:
    """Copies the package; returns the destination, or None when there is no checkout to copy from."""
    src = find_checkout(reference)
    if src is None:
        if verbose:
            print("make_ref: no reference checkout found; oracle/_ref left as it is "
                  f"({'present' if (DEST / 'nncf').exists() else 'absent'})")
        return DEST if (DEST / "nncf").exists() else None
    pkg = src / "src" / "nncf"
    out = DEST / "nncf"
    if out.exists() and _same_tree(pkg, out):
        if verbose:
            print(f"make_ref: {out} is up to date")
        return DEST
    if out.exists():
        shutil.rmtree(out)
    DEST.mkdir(parents=True, exist_ok=True)
    shutil.copytree(pkg, out, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    (DEST / "SOURCE.txt").write_text(
        "Unmodified copy of src/nncf of openvinotoolkit/nncf made by oracle/make_ref.py.\n"
        "Not product source; not tracked by git.\n")
    if verbose:
        n = sum(1 for _ in out.rglob("*.py"))
        print(f"make_ref: copied {n} python files to {out}")
    return DEST


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None, help="checkout of the reference (the directory that holds src/nncf)")
    ns = ap.parse_args()
    sys.exit(0 if make_ref(ns.reference) is not None else 1)
