"""Full validation of a plan/run pair, phase by phase, without launching model workers:

    python -m rpeg_b200.runtime.validate_full --config run.yaml [--backend engine] [--report report.json]

  1 input            strict run schema, plan hash, run-vs-plan agreement
  2 unroll           the algorithm graph unrolled over ``training.max_steps`` (publication edges, staleness)
  3 lower            explicit transfers, quantile phases, fusion groups; memory feasibility per GPU
  4 runtime graph    dependencies, workers, resource keys, recorded dispatch order, acyclicity
  5 metadata run     asynchronous execution with the metadata backend, trace verification, alert rules
  6 backend run      (optional, ``--backend engine``) the same graph on the GPU engine

Each phase reports ``ok`` plus a few facts; the first failing phase stops the run. Exit code 0 if all
requested phases pass, 2 on configuration errors, 1 on execution errors.
Reference: RPEG/runtime/validate_full.py:98-449.
"""
from __future__ import annotations

import argparse
import json
import sys
import tempfile
import time
from pathlib import Path
from typing import Any, Dict, List, Optional

from ..passes.lower import ExecNodeType
from .compiler import compile_runtime_plan
from .errors import RuntimeConfigError, RuntimeExecutionError
from .executor import MetadataOnlyOperationHandler, RuntimeExecutor
from .metrics import evaluate_alerts, summarize_trace
from .schema import OptimizedPlan, RuntimeRunConfig
from .trace import RuntimeTraceWriter, read_trace
from .verification import verify_runtime_trace

REPORT_SCHEMA = "rpeg.full_validation.v1"


def _phase(report: Dict[str, Any], name: str, fn) -> bool:
    t0 = time.perf_counter()
    try:
        facts = fn() or {}
        report["phases"].append({"phase": name, "ok": True, "seconds": time.perf_counter() - t0, **facts})
        return True
    except (RuntimeConfigError, RuntimeExecutionError, ValueError, KeyError) as exc:
        report["phases"].append({"phase": name, "ok": False, "seconds": time.perf_counter() - t0,
                                 "error": f"{type(exc).__name__}: {exc}", "config_error": isinstance(exc, (RuntimeConfigError, ValueError, KeyError))})
        return False


def validate_full(config_path, *, backend: Optional[str] = None, work_dir=None) -> Dict[str, Any]:
    report: Dict[str, Any] = {"schema_version": REPORT_SCHEMA, "config": str(config_path), "phases": []}
    box: Dict[str, Any] = {}

    def p_input():
        run = RuntimeRunConfig.load(config_path)
        plan = OptimizedPlan.load(run.resolve(run.optimized_plan.path), run.optimized_plan.expected_hash)
        box["run"] = run
        return {"run_id": run.run_id, "algorithm": run.algorithm.name, "plan_hash": plan.plan_hash, "vertices": len(plan.vertices),
                "has_schedule": plan.schedule is not None}

    def p_unroll():
        c = compile_runtime_plan(box["run"], dry_run=True)
        box["compiled"] = c
        return {"steps": box["run"].training.max_steps, "unrolled_nodes": len(c.unrolled.nodes),
                "data_edges": len(c.unrolled.data_edges), "publication_edges": len(c.unrolled.pub_edges), "tau": {m.value: int(t) for m, t in c.config.rpeg.tau.items()}}

    def p_lower():
        c = box["compiled"]
        kinds: Dict[str, int] = {}
        for n in c.lowered.nodes:
            kinds[n.kind.value] = kinds.get(n.kind.value, 0) + 1
        split = sum(1 for n in c.lowered.nodes if n.n_seqs is not None)
        return {"lowered_nodes": len(c.lowered.nodes), "lowered_edges": len(c.lowered.edges), "by_kind": kinds,
                "quantile_split_nodes": split, "fusion_groups": len({n.fusion_group for n in c.lowered.nodes if n.fusion_group}),
                "transfer_payload_bytes": int(sum(n.payload_in_bytes for n in c.lowered.nodes if n.kind is not ExecNodeType.OP))}

    def p_graph():
        g = box["compiled"].runtime_graph()
        box["graph"] = g
        pos = {n: i for i, n in enumerate(g.topological_order)}
        for nid, n in g.nodes.items():
            for d in n.dependencies:
                if pos[d] >= pos[nid]:
                    raise RuntimeConfigError(f"runtime order violates dependency {d}->{nid}")
            if n.kind is ExecNodeType.OP and not any(k.startswith("worker:") for k in n.resource_keys):
                raise RuntimeConfigError(f"operator {nid} holds no worker")
        gpus = {k for n in g.nodes.values() for k in n.resource_keys if k.startswith("gpu:")}
        return {"nodes": len(g.nodes), "edges": len(g.edges), "workers": len(box["compiled"].workers), "gpus_used": len(gpus),
                "recorded_order": box["compiled"].execution_order is not None}

    def p_metadata():
        c, g = box["compiled"], box["graph"]
        d = Path(work_dir) if work_dir else Path(tempfile.mkdtemp(prefix="rpeg_validate_"))
        d.mkdir(parents=True, exist_ok=True)
        with RuntimeTraceWriter(d / "metadata_trace.jsonl", run_id=c.run_config.run_id) as tw:
            RuntimeExecutor(g, run_id=c.run_config.run_id, handler=MetadataOnlyOperationHandler(c), trace=tw,
                            node_timeout_s=c.run_config.runtime.node_timeout_s).run()
        events = read_trace(d / "metadata_trace.jsonl")
        rep = verify_runtime_trace(c, g, events)
        alerts = evaluate_alerts(summarize_trace(events), c.run_config.monitoring.alert_rules, rep)
        if alerts["status"] == "critical":
            raise RuntimeExecutionError("alerts: " + "; ".join(a["message"] for a in alerts["alerts"]))
        return {"events": len(events), "verified_nodes": rep["verified_nodes"], "alerts": alerts["status"], "trace": str(d / "metadata_trace.jsonl")}

    def p_backend():
        from .run import execute_compiled
        res = execute_compiled(box["compiled"], backend)
        if res["error"] is not None:
            raise RuntimeExecutionError(res["error"])
        if not res["verification"]["ok"]:
            raise RuntimeExecutionError("; ".join(res["verification"]["errors"][:5]))
        return {"backend": backend, "events": res["events"], "attempts": res["attempts"], "summary": res["summary"]}

    phases = [("input", p_input), ("unroll", p_unroll), ("lower", p_lower), ("runtime_graph", p_graph), ("metadata_execution", p_metadata)]
    if backend and backend != "metadata":
        phases.append(("backend_execution", p_backend))
    ok = True
    for name, fn in phases:
        if not _phase(report, name, fn):
            ok = False
            break
    report["ok"] = ok
    return report


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="Validate a run file phase by phase")
    ap.add_argument("--config", required=True)
    ap.add_argument("--backend", default=None, choices=(None, "metadata", "engine"))
    ap.add_argument("--report", default=None)
    ap.add_argument("--work-dir", default=None)
    args = ap.parse_args(argv)
    report = validate_full(args.config, backend=args.backend, work_dir=args.work_dir)
    text = json.dumps(report, indent=2, default=str)
    if args.report:
        Path(args.report).write_text(text)
    print(text)
    if report["ok"]:
        return 0
    return 2 if report["phases"][-1].get("config_error") else 1


if __name__ == "__main__":
    sys.exit(main())
