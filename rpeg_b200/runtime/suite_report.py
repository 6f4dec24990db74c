"""Aggregate the JSON reports of the validation tools into one verdict:

    python -m rpeg_b200.runtime.suite_report --inputs env.json dist.json validate.json metrics/summary.json --output suite.json

Understands the schemas written by ``environment_check``, ``distributed_validate``,
``validate_full``, ``collective_benchmark``, ``cost_calibration``, the runtime summary and alert
report, and a ``bench.py`` line; anything else is listed as ``unknown`` and counted as a failure only
with ``--strict``. Output ``rpeg.suite_report.v1``; exit code 0 only if every recognised report passes.
Reference: RPEG/runtime/suite_report.py:85-136.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path
from typing import Any, Dict, List, Optional

SCHEMA = "rpeg.suite_report.v1"


def classify(doc: Dict[str, Any]) -> Dict[str, Any]:
    sv = str(doc.get("schema_version", ""))
    if sv in ("rpeg.environment_check.v1", "rpeg.distributed_validation.v1", "rpeg.full_validation.v1"):
        detail = {}
        if sv == "rpeg.full_validation.v1":
            detail = {"phases": [p["phase"] for p in doc.get("phases", ()) if p.get("ok")],
                      "failed": [p for p in doc.get("phases", ()) if not p.get("ok")]}
        if sv == "rpeg.environment_check.v1":
            detail = {"failed": [c["name"] for c in doc.get("checks", ()) if c.get("required") and not c.get("ok")]}
        return {"kind": sv.split(".")[1], "ok": bool(doc.get("ok")), "detail": detail}
    if sv == "rpeg.engine_validate.v1":
        return {"kind": "engine_validate", "ok": bool(doc.get("ok")),
                "detail": {"world": doc.get("world"), "failed": [c["name"] for c in doc.get("checks", ()) if not c.get("ok")], "error": doc.get("error")}}
    if sv == "rpeg.cluster_contract.v1":
        return {"kind": "cluster_contract", "ok": bool(doc.get("performance_comparable")),
                "detail": {"nodes": doc.get("nodes"), "reasons": doc.get("non_comparable_reasons", [])}}
    if sv == "rpeg.runtime_alerts.v1":
        return {"kind": "alerts", "ok": doc.get("status") != "critical", "detail": {"status": doc.get("status"), "alerts": len(doc.get("alerts", ()))}}
    if sv == "rpeg.runtime_summary.v1":
        ok = doc.get("nodes_failed", 0) == 0 and doc.get("nodes_incomplete", 0) == 0 and doc.get("nonfinite_losses", 0) == 0
        return {"kind": "runtime_summary", "ok": ok, "detail": {k: doc.get(k) for k in ("nodes_finished", "nodes_failed", "wall_time_s", "logical_steps")}}
    if sv == "rpeg.collective_benchmark.v1":
        rows = doc.get("rows", ())
        return {"kind": "collective_benchmark", "ok": bool(rows) and bool((doc.get("gate") or {}).get("ok", True)), "detail": {"world": doc.get("world"),
                "all_reduce_busbw_gbs": max((r.get("nccl_all_reduce_busbw_gbs", 0) for r in rows), default=0)}}
    if sv == "rpeg.cost_calibration.v1":
        return {"kind": "cost_calibration", "ok": doc.get("matched_nodes", 0) > 0, "detail": doc.get("hardware", {})}
    if "metric" in doc and "value" in doc:
        return {"kind": "bench", "ok": float(doc.get("value") or 0) > 0 and int(doc.get("gpu_launches") or 0) > 0,
                "detail": {k: doc.get(k) for k in ("metric", "value", "unit", "n_gpus", "ms_per_step")}}
    if doc.get("impl") == "reference" and "unavailable" in doc:
        return {"kind": "bench_reference", "ok": True, "detail": {"unavailable": doc["unavailable"]}}
    return {"kind": "unknown", "ok": None, "detail": {"keys": sorted(doc)[:10]}}


def aggregate(paths: List[str], strict: bool = False) -> Dict[str, Any]:
    items = []
    for p in paths:
        try:
            text = Path(p).read_text().strip()
            doc = json.loads(text.splitlines()[-1] if not text.startswith("{\n") and "\n" in text and text.splitlines()[-1].startswith("{") else text)
            items.append({"path": str(p), **classify(doc)})
        except Exception as exc:
            items.append({"path": str(p), "kind": "unreadable", "ok": False, "detail": {"error": str(exc)}})
    bad = [i for i in items if i["ok"] is False or (strict and i["ok"] is None)]
    return {"schema_version": SCHEMA, "ok": not bad, "reports": len(items), "failed": [i["path"] for i in bad], "items": items}


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--inputs", nargs="+", required=True)
    ap.add_argument("--output", default=None)
    ap.add_argument("--strict", action="store_true")
    args = ap.parse_args(argv)
    rep = aggregate(args.inputs, args.strict)
    if args.output:
        Path(args.output).write_text(json.dumps(rep, indent=1, default=str))
    print(json.dumps(rep, indent=1, default=str))
    return 0 if rep["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
