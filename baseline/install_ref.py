"""Puts a runnable copy of the reference under ``baseline/_ref`` for ``bench.py --impl reference``.

    python baseline/install_ref.py [--source <reference source tree>] [--force]

The reference is pure Python and is run from its source tree (``PYTHONPATH=<tree>/RPEG:<tree>``, as its own
runtime README does); its build backend (hatchling) is not available offline, so ``pip install`` of it
fails and is not needed. The shipped tree does not import as published; ``baseline/ref_import_fixes.patch``
holds the five one-line repairs (a misspelt class name, an unbalanced bracket in an annotation, two missing
imports, a misspelt variable) and nothing else is changed. The copy leaves out ``paper/`` (a results archive
and its plotting script) and ``.git``.
"""
from __future__ import annotations

import argparse
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"
PATCH = HERE / "ref_import_fixes.patch"
MARK = DEST / ".installed"


def install(source: Path, force: bool = False) -> Path:
    if MARK.exists() and not force:
        return DEST
    if not (source / "RPEG").is_dir():
        raise FileNotFoundError(f"{source} does not look like the reference tree (no RPEG/ directory)")
    if DEST.exists():
        shutil.rmtree(DEST)
    shutil.copytree(source, DEST, ignore=shutil.ignore_patterns(".git", "paper", "__pycache__"))
    res = subprocess.run(["patch", "-p1", "-d", str(DEST), "-i", str(PATCH)], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"patch failed:\n{res.stdout}\n{res.stderr}")
    MARK.write_text(f"copied from {source}; patched with {PATCH.name}\n")
    return DEST


def env_for_reference() -> dict:
    """Environment of a subprocess that runs the reference: its package roots first, then the matplotlib
    stand-in (the image has no matplotlib and ``pipeline.py`` imports it unconditionally)."""
    import os
    env = dict(os.environ)
    roots = [str(DEST / "RPEG"), str(DEST), str(HERE / "stubs")]
    env["PYTHONPATH"] = os.pathsep.join(roots + ([env["PYTHONPATH"]] if env.get("PYTHONPATH") else []))
    env["PYTHONDONTWRITEBYTECODE"] = "1"
    return env


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--source", default="/root/reference")
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args()
    dest = install(Path(args.source), args.force)
    print(f"reference copy ready at {dest}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
