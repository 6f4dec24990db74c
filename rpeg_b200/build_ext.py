"""In-tree build of the native kernels: ``rpeg_b200/librpeg_kernels.so`` (sm_100a only).

Each ``csrc/*.cu`` is compiled by nvcc (cross-compiles without a GPU) into an object next to the
source and the objects are linked into one shared library that ``rpeg_b200.ops._lib`` loads with
ctypes. Objects are rebuilt only when their source or a header is newer.

Run ``python -m rpeg_b200.build_ext`` (add ``--verbose`` for ptxas register/spill output).
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "librpeg_kernels.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--use_fast_math",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put it on PATH)")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale(obj: Path, src: Path, headers: list[Path]) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    return any(p.stat().st_mtime > t for p in [src, *headers])


def _compile(src: Path, verbose: bool) -> tuple[Path, str]:
    obj = src.with_suffix(".o")
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    return obj, res.stderr


def build(verbose: bool = False, force: bool = False) -> Path:
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh"))
    srcs = sources()
    todo = [s for s in srcs if force or _stale(s.with_suffix(".o"), s, headers)]
    logs: list[str] = []
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 4)) as ex:
            for obj, log in ex.map(lambda s: _compile(s, verbose), todo):
                logs.append(f"== {obj.name}\n{log}")
    objs = [s.with_suffix(".o") for s in srcs]
    if todo or not LIB.exists() or any(o.stat().st_mtime > LIB.stat().st_mtime for o in objs):
        cmd = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    if verbose:
        print("\n".join(logs))
    return LIB


if __name__ == "__main__":
    path = build(verbose="--verbose" in sys.argv, force="--force" in sys.argv)
    print(path)
