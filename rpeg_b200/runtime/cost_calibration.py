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


def calibrate_costs(compiled, events: Sequence[dict], hw=None) -> Dict[str, Any]:
    run = compiled.run_config
    hw = hw or b200_nvswitch(mem=float(run.hardware.memory_per_gpu_bytes))
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
    args = ap.parse_args(argv)
    try:
        compiled = compile_runtime_plan(args.config, dry_run=True)
    except RuntimeConfigError as exc:
        print(f"runtime error: {exc}", file=sys.stderr)
        return 2
    rep = calibrate_costs(compiled, read_trace(args.trace))
    if args.output:
        dump_mapping(rep["hardware"], args.output)
    print(json.dumps({k: v for k, v in rep.items() if k != "nodes"}, indent=2))
    return 0 if rep["matched_nodes"] else 1


if __name__ == "__main__":
    sys.exit(main())
