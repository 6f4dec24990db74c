"""Run a planned job:

    python -m rpeg_b200.runtime.run --config run.yaml --dry-run                  # compile only, print the summary
    python -m rpeg_b200.runtime.run --config run.yaml --execute-graph-metadata   # execute the graph contracts, no tensors
    python -m rpeg_b200.runtime.run --config run.yaml                            # execute with runtime.default_backend

Every mode compiles the run/plan pair first; configuration and compilation errors are reported as
``runtime error: ...`` with exit code 2, execution errors with exit code 1. An executed run writes
its JSONL trace, verifies it against the compiled graph and writes the summary, the Prometheus text,
the alert report and the dashboard to the paths of the ``monitoring`` section.
Reference: RPEG/runtime/run.py:86-149.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Any, Dict, List, Optional

from .compiler import CompiledRuntimePlan, compile_runtime_plan
from .errors import RuntimeConfigError, RuntimeExecutionError
from .executor import MetadataOnlyOperationHandler
from .metrics import write_runtime_summary_for_run
from .recovery import run_with_replay
from .trace import RuntimeTraceWriter, read_trace
from .verification import verify_runtime_trace


def execute_compiled(compiled: CompiledRuntimePlan, backend: str, *, trace_path=None) -> Dict[str, Any]:
    run = compiled.run_config
    graph = compiled.runtime_graph()
    trace_file = run.resolve(trace_path or run.runtime.trace_path)
    # One process per GPU runs the same graph: rank 0 owns the run's trace, summary and alert files, the other
    # ranks keep their own trace next to it (``run.rank3.jsonl``) and verify it without writing summaries.
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    secondary = backend == "engine" and world > 1 and rank > 0
    if secondary:
        trace_file = trace_file.with_name(f"{trace_file.stem}.rank{rank}{trace_file.suffix}")
    if backend == "metadata":
        make_handler = lambda attempt: MetadataOnlyOperationHandler(compiled)
    elif backend == "engine":
        from .engine_backend import make_engine_handler_factory
        make_handler = make_engine_handler_factory(compiled)
    else:
        raise RuntimeConfigError(f"unknown backend {backend!r}")
    with RuntimeTraceWriter(trace_file, run_id=run.run_id) as tw:
        for node in ("runtime.workers.start", "runtime.workers.initialize", "runtime.weights.publish_initial"):
            tw.emit(node, "start", counters={"workers": len(compiled.workers)})
            tw.emit(node, "finish", counters={"workers": len(compiled.workers)})
        error: Optional[Exception] = None
        outcome: Dict[str, Any] = {}
        try:
            outcome = run_with_replay(compiled, graph, make_handler, tw, node_timeout_s=run.runtime.node_timeout_s)
        except RuntimeExecutionError as exc:
            error = exc
    events = read_trace(trace_file)
    report = verify_runtime_trace(compiled, graph, events, raise_on_error=False,
                                  completed_before=outcome.get("completed_before", ()) if run.checkpoints.resume_from else ())
    if secondary:
        return {"run_id": run.run_id, "backend": backend, "rank": rank, "trace": str(trace_file), "events": len(events),
                "verification": report, "alerts": None, "attempts": outcome.get("attempts"),
                "error": None if error is None else str(error), "summary": {}}
    written = write_runtime_summary_for_run(run, events, verification=report,
                                            extra={"backend": backend, "attempts": outcome.get("attempts"),
                                                   "restored_step": outcome.get("restored_step")})
    return {"run_id": run.run_id, "backend": backend, "trace": str(trace_file), "events": len(events), "verification": report,
            "alerts": written["alerts"]["status"], "attempts": outcome.get("attempts"), "error": None if error is None else str(error),
            "summary": {k: written["summary"].get(k) for k in ("nodes_finished", "nodes_failed", "wall_time_s", "logical_steps",
                                                               "replay_attempts", "checkpoint_saves")}}


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="Compile and execute an RPEG run file")
    ap.add_argument("--config", required=True)
    ap.add_argument("--dry-run", action="store_true", help="compile and print the compilation summary")
    ap.add_argument("--execute-graph-metadata", action="store_true", help="execute the graph with the metadata backend")
    ap.add_argument("--trace", default=None, help="trace path (default: runtime.trace_path of the run file)")
    args = ap.parse_args(argv)
    try:
        compiled = compile_runtime_plan(args.config, dry_run=args.dry_run)
        if args.dry_run or (compiled.run_config.runtime.dry_run and not args.execute_graph_metadata):
            print(json.dumps(compiled.summary(), indent=2, default=str))
            return 0
        backend = "metadata" if args.execute_graph_metadata else compiled.run_config.runtime.default_backend
        result = execute_compiled(compiled, backend, trace_path=args.trace)
    except RuntimeConfigError as exc:
        print(f"runtime error: {exc}", file=sys.stderr)
        return 2
    print(json.dumps(result, indent=2, default=str))
    if result["error"] is not None:
        print(f"execution error: {result['error']}", file=sys.stderr)
        return 1
    return 0 if result["verification"]["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
