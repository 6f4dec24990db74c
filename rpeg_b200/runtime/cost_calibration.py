"""Fit the cost model's scale factors to a measured run.

    python -m rpeg_b200.runtime.cost_calibration --config run.yaml --trace traces/run.jsonl --output hw_scales.yaml

For every node of the compiled graph the analytical duration (the list scheduler's cost model on the
run's hardware) is set against the measured duration in the trace. Per class of node the multiplicative
residual is fitted through the origin (least squares on ``measured = scale * predicted``):
``op_generation_scale``, ``op_inference_scale``, ``op_training_scale``, ``weight_comm_scale``,
``reshard_scale`` and an additive ``activation_comm_overhead_s`` (median residual of activation
transfers). The output is a flat hardware fragment to merge with ``pipeline.py --hw`` or the job
file's ``hardware`` section. Reference: RPEG/runtime/cost_calibration.py:60-275.
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
from typing import Any, Dict, List, Optional, Sequence, Tuple

from ..analytic.cost import NodeCostModel
from ..analytic.hardware import b200_nvswitch
from ..passes.lower import ExecNodeType
from .compiler import compile_runtime_plan, memory_policy_from_run
from .errors import RuntimeConfigError
from .io import dump_mapping
from .trace import read_trace

SCHEMA = "rpeg.cost_calibration.v1"


def measured_durations(events: Sequence[dict]) -> Dict[str, float]:
    """Seconds per node id from the last successful start/finish pair (``duration_s`` counter if present)."""
    starts: Dict[str, float] = {}
    out: Dict[str, float] = {}
    for e in events:
        if e.get("event") == "start":
            starts[e["node_id"]] = float(e["timestamp"])
        elif e.get("event") == "finish" and e.get("status") == "ok" and e["node_id"] in starts:
            c = e.get("counters") or {}
            out[e["node_id"]] = float(c.get("duration_s", float(e["timestamp"]) - starts[e["node_id"]]))
    return out


def fit_scale(pairs: Sequence[Tuple[float, float]]) -> Optional[float]:
    """argmin_s sum (m - s p)^2 = sum(m p) / sum(p p)."""
    den = sum(p * p for p, _ in pairs)
    return sum(p * m for p, m in pairs) / den if den > 0 else None


def hardware_for_run(run, files: Sequence[str] = ()):
    """The B200 preset with the run's memory size, overlaid with hardware files in order (a ``calibrate.py``
    output, then fragments written by earlier fits) and, for the engine backend, with the generator's limits from
    the run file (slots, paged KV pool) unless a file already sets them."""
    import yaml
    from ..analytic.hardware import Hardware
    hw = b200_nvswitch(mem=float(run.hardware.memory_per_gpu_bytes))
    names = set(Hardware.field_names())
    for path in files:
        with open(path) as fh:
            data = yaml.safe_load(fh) or {}
        upd = {k: (v if k == "fabric" else float(v)) for k, v in data.items() if k in names and k != "memory_per_gpu"}
        hw = hw.with_updates(**upd)
    rt = getattr(run, "runtime", None)
    extra = {}
    slots = getattr(rt, "gen_slots", None) if rt is not None else None
    if slots and not hw.gen_max_concurrency > 0:
        extra["gen_max_concurrency"] = float(slots)
    kvb = float(getattr(run.hardware, "kv_cache_budget_bytes", 0) or 0)
    if kvb > 0 and not hw.gen_kv_budget_bytes > 0:
        extra["gen_kv_budget_bytes"] = kvb
    return hw.with_updates(**extra) if extra else hw


def prediction_error(rep: Dict[str, Any]) -> Dict[str, Any]:
    """Per node class and overall: sum of predicted against sum of measured seconds (signed relative error)."""
    acc: Dict[str, List[float]] = {}
    for r in rep["nodes"]:
        a = acc.setdefault(r["class"], [0.0, 0.0])
        a[0] += r["predicted_s"]
        a[1] += r["measured_s"]
    out = {k: {"predicted_s": p, "measured_s": m, "relative_error": (p - m) / m if m > 0 else None} for k, (p, m) in acc.items()}
    tp, tm = sum(p for p, _ in acc.values()), sum(m for _, m in acc.values())
    out["total"] = {"predicted_s": tp, "measured_s": tm, "relative_error": (tp - tm) / tm if tm > 0 else None}
    return out


def calibrate_costs(compiled, events: Sequence[dict], hw=None) -> Dict[str, Any]:
    run = compiled.run_config
    hw = hw or hardware_for_run(run)
    pol = memory_policy_from_run(run)
    cost = NodeCostModel(hw, compiled.model_suite, compiled.workload, optimizer_stage=pol.optimizer_stage,
                         activation_checkpointing=pol.activation_checkpointing)
    measured = measured_durations(events)
    groups: Dict[str, List[Tuple[float, float]]] = {"GEN": [], "INF": [], "TRAIN": [], "weight": [], "reshard": [], "activation": []}
    rows = []
    for n in compiled.lowered.nodes:
        if n.id not in measured:
            continue
        pred, meas = float(cost.time(n)), measured[n.id]
        if n.kind is ExecNodeType.OP:
            key = n.role.value
        elif n.kind is ExecNodeType.RESHARD:
            key = "reshard"
        else:
            key = "weight" if str(n.label or "").startswith("W_") else "activation"
        groups[key].append((pred, meas))
        rows.append({"node_id": n.id, "class": key, "predicted_s": pred, "measured_s": meas})
    names = {"GEN": "op_generation_scale", "INF": "op_inference_scale", "TRAIN": "op_training_scale", "weight": "weight_comm_scale",
             "reshard": "reshard_scale"}
    fragment: Dict[str, float] = {}
    stats: Dict[str, Any] = {}
    for key, field in names.items():
        s = fit_scale(groups[key])
        if s is not None and s > 0:
            fragment[field] = getattr(hw, field) * s
            resid = [m - s * p for p, m in groups[key]]
            stats[key] = {"nodes": len(groups[key]), "scale": s, "rmse_s": (sum(r * r for r in resid) / len(resid)) ** 0.5}
    act = [m - p for p, m in groups["activation"]]
    if act:
        fragment["activation_comm_overhead_s"] = max(0.0, hw.activation_comm_overhead_s + statistics.median(act))
        stats["activation"] = {"nodes": len(act), "median_residual_s": statistics.median(act)}
    return {"schema_version": SCHEMA, "run_id": run.run_id, "matched_nodes": len(rows), "hardware": fragment, "classes": stats, "nodes": rows}


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="Fit cost-model scales to a measured trace")
    ap.add_argument("--config", required=True)
    ap.add_argument("--trace", required=True)
    ap.add_argument("--output", default=None, help="hardware fragment (yaml or json)")
    ap.add_argument("--report", default=None, help="write the full report (one row per node with predicted and measured seconds) "
                    "as JSON, the input of experiments/plot_cost_model_validation.py")
    ap.add_argument("--hw", action="append", default=[], help="hardware file(s) laid over the B200 preset before predicting: "
                    "a calibrate.py output and/or a fragment from an earlier fit (validation of that fit on this run)")
    args = ap.parse_args(argv)
    try:
        compiled = compile_runtime_plan(args.config, dry_run=True)
    except RuntimeConfigError as exc:
        print(f"runtime error: {exc}", file=sys.stderr)
        return 2
    rep = calibrate_costs(compiled, read_trace(args.trace), hardware_for_run(compiled.run_config, args.hw))
    rep["prediction_error"] = prediction_error(rep)
    if args.report:
        with open(args.report, "w") as fh:
            json.dump(rep, fh, indent=1)
    if args.output:
        dump_mapping(rep["hardware"], args.output)
    print(json.dumps({k: v for k, v in rep.items() if k != "nodes"}, indent=2))
    return 0 if rep["matched_nodes"] else 1


if __name__ == "__main__":
    sys.exit(main())
