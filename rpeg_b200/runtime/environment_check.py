"""Preflight: does this machine have what a run needs?

    python -m rpeg_b200.runtime.environment_check [--config run.yaml] [--json]

Checks Python packages, the CUDA toolchain, the in-tree kernel library (present, loadable, exports the
C ABI), the GPUs (count, name, memory, compute capability 10.x, peer access between every pair) and,
with ``--config``, that the node has the GPUs and the memory the run file plans for. Read-only: no
GPU setting is touched. Every check yields ``{name, ok, detail}``; exit code 0 only if all required
checks pass. Reference: RPEG/runtime/environment_check.py:80-189. The per-node health line and the
cluster contract of a Slurm allocation are in ``runtime/slurm_preflight.py``.
"""
from __future__ import annotations

import argparse
import importlib
import json
import shutil
import sys
from pathlib import Path
from typing import Any, Dict, List, Optional

SCHEMA = "rpeg.environment_check.v1"
REQUIRED_PACKAGES = ("torch", "numpy", "yaml")
OPTIONAL_PACKAGES = ("pytest",)


def _check(name: str, ok: bool, detail: Any, required: bool = True) -> Dict[str, Any]:
    return {"name": name, "ok": bool(ok), "required": required, "detail": detail}


def run_checks(config: Optional[str] = None, need_gpu: bool = True) -> Dict[str, Any]:
    out: List[Dict[str, Any]] = []
    for pkg in REQUIRED_PACKAGES + OPTIONAL_PACKAGES:
        try:
            m = importlib.import_module(pkg)
            out.append(_check(f"package:{pkg}", True, getattr(m, "__version__", "?"), pkg in REQUIRED_PACKAGES))
        except Exception as exc:
            out.append(_check(f"package:{pkg}", False, str(exc), pkg in REQUIRED_PACKAGES))
    out.append(_check("tool:nvcc", shutil.which("nvcc") is not None, shutil.which("nvcc"), required=False))
    lib_path = Path(__file__).resolve().parents[1] / "librpeg_kernels.so"
    out.append(_check("kernels:built", lib_path.exists(), str(lib_path)))
    try:
        from ..ops._lib import _SIGNATURES, lib
        h = lib()
        missing = [s for s in _SIGNATURES if not hasattr(h, s)]
        out.append(_check("kernels:abi", not missing, {"entries": len(_SIGNATURES), "missing": missing}))
    except Exception as exc:
        out.append(_check("kernels:abi", False, str(exc)))
    gpus: List[Dict[str, Any]] = []
    try:
        import torch
        n = torch.cuda.device_count() if torch.cuda.is_available() else 0
        out.append(_check("gpu:visible", n > 0, n, required=need_gpu))
        for i in range(n):
            p = torch.cuda.get_device_properties(i)
            gpus.append({"index": i, "name": p.name, "memory_bytes": p.total_memory, "capability": [p.major, p.minor], "sms": p.multi_processor_count})
            out.append(_check(f"gpu:{i}:capability", p.major == 10, f"{p.major}.{p.minor} ({p.name})", required=need_gpu))
        bad = [(a, b) for a in range(n) for b in range(n) if a != b and not torch.cuda.can_device_access_peer(a, b)]
        if n > 1:
            out.append(_check("gpu:peer_access", not bad, {"pairs_without_access": bad}))
        out.append(_check("distributed:nccl", torch.distributed.is_nccl_available(), None, required=need_gpu))
        out.append(_check("distributed:gloo", torch.distributed.is_gloo_available(), None))
    except Exception as exc:
        out.append(_check("gpu:query", False, str(exc), required=need_gpu))
    if config:
        try:
            from .schema import RuntimeRunConfig
            run = RuntimeRunConfig.load(config)
            want = run.device_space.racks * run.device_space.nodes_per_rack * run.device_space.gpus_per_node
            out.append(_check("run:gpu_count", len(gpus) >= want, {"planned": want, "visible": len(gpus)}, required=need_gpu))
            short = [g["index"] for g in gpus if g["memory_bytes"] < run.hardware.memory_per_gpu_bytes * 0.95]
            out.append(_check("run:gpu_memory", not short, {"planned_bytes": run.hardware.memory_per_gpu_bytes, "too_small": short}, required=need_gpu))
        except Exception as exc:
            out.append(_check("run:config", False, str(exc)))
    ok = all(c["ok"] for c in out if c["required"])
    return {"schema_version": SCHEMA, "ok": ok, "checks": out, "gpus": gpus}


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default=None)
    ap.add_argument("--no-gpu", action="store_true", help="GPU checks are informational (planner-only machines)")
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)
    rep = run_checks(args.config, need_gpu=not args.no_gpu)
    if args.json:
        print(json.dumps(rep, indent=1, default=str))
    else:
        for c in rep["checks"]:
            mark = "ok  " if c["ok"] else ("FAIL" if c["required"] else "warn")
            print(f"[{mark}] {c['name']}: {c['detail']}")
        print("environment " + ("ok" if rep["ok"] else "NOT ok"))
    return 0 if rep["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
