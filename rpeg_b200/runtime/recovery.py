"""Bounded graph replay: run the runtime graph, and when a node fails, restore the newest usable
interval checkpoint and execute only the suffix of the graph that the checkpoint does not cover.

A logical step is *closed* once every TRAIN node of that step has finished; a checkpoint is written
at closed steps that are multiples of ``checkpoints.interval_steps`` (and at the end, if
``save_final``). After a failure, attempt ``a+1`` (``monitoring.graph_replay_retries`` extra
attempts at most) emits a ``replay`` trace event, picks the newest verified checkpoint, emits
``recover`` with the restored step and weight versions, and runs the subgraph of nodes whose logical
step is greater than the restored one; without a usable checkpoint it restarts from the beginning.
There is no re-planning and no change of allocation. Reference: RPEG/runtime/recovery.md:31-71,
RPEG/runtime/algorithms/megatron_ppo_graph.py:1033-1103 (completion hook), :3268-3362 (replay loop).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Set

from . import checkpoint as ckpt
from .errors import RuntimeExecutionError
from .executor import RuntimeExecutionContext, RuntimeExecutor, model_name
from .graph import RuntimeGraph, RuntimeNodeSpec, suffix_node_ids
from .trace import RuntimeTraceWriter


class InjectedFailure(RuntimeExecutionError):
    """Raised on the host by the test hooks of ``monitoring.test_inject_failure_*``."""


@dataclass
class StepTracker:
    """Which logical steps have all their TRAIN nodes finished."""
    graph: RuntimeGraph
    train_nodes: Dict[int, Set[str]] = field(default_factory=dict)
    finished: Set[str] = field(default_factory=set)
    closed: Set[int] = field(default_factory=set)

    def __post_init__(self):
        for nid, n in self.graph.nodes.items():
            if n.role == "TRAIN" and n.logical_step is not None:
                self.train_nodes.setdefault(int(n.logical_step), set()).add(nid)

    def node_done(self, node: RuntimeNodeSpec) -> Optional[int]:
        """Record a finished node; returns the step it closed, if any."""
        self.finished.add(node.node_id)
        s = node.logical_step
        if node.role != "TRAIN" or s is None or int(s) in self.closed:
            return None
        if self.train_nodes.get(int(s), set()) <= self.finished:
            self.closed.add(int(s))
            return int(s)
        return None


def suffix_graph(graph: RuntimeGraph, restored_step: int) -> RuntimeGraph:
    """Nodes that still have to run after restoring the state at the end of ``restored_step``."""
    return graph.subgraph(suffix_node_ids(graph, restored_step))


class CheckpointingHook:
    """Wraps a handler: forwards execution, tracks step closure, saves checkpoints through the
    handler's ``save_checkpoint(step, path, kind)`` (metadata handlers write manifests only) and
    injects the configured test failure after a checkpoint step."""

    def __init__(self, inner, graph: RuntimeGraph, run_config, trace: Optional[RuntimeTraceWriter], attempt: int,
                 latest_versions: Optional[Dict[str, int]] = None):
        self.inner, self.graph, self.run, self.trace, self.attempt = inner, graph, run_config, trace, attempt
        self.tracker = StepTracker(graph)
        self.latest = dict(latest_versions or {})
        self.saved_steps: List[int] = []

    def __getattr__(self, name):            # select_batch / execute_batch / anything else the handler offers
        return getattr(self.inner, name)

    async def execute(self, node, context):
        m = self.run.monitoring
        if (m.test_inject_failure_node_contains and m.test_inject_failure_attempt == self.attempt
                and m.test_inject_failure_node_contains in node.node_id):
            raise InjectedFailure(f"injected failure at node {node.node_id} (attempt {self.attempt})")
        return await self.inner.execute(node, context)

    def output_dir(self):
        return self.run.resolve(self.run.checkpoints.output_dir)

    def _tau(self) -> Dict[str, int]:
        comp = getattr(self.inner, "compiled", None)
        if comp is None:
            return {}
        return {model_name(m.value): int(t) for m, t in comp.config.rpeg.tau.items()}

    def save(self, step: int, kind: str) -> None:
        out = self.output_dir()
        name = "final" if kind == "final" else f"step_{step}"
        path = out / name
        path.mkdir(parents=True, exist_ok=True)
        if self.trace is not None:
            self.trace.emit("runtime.checkpoint.save", "start", step=step, counters={"name": name, "kind": kind})
        saver = getattr(self.inner, "save_checkpoint", None)
        # every rank writes its own shards (the handler synchronises the ranks around that); the manifest, the index
        # entry and the pruning of old checkpoints are the work of ONE process, or the ranks race on the same files
        info = saver(step, path, kind) if saver is not None else {"workers": [], "bytes": 0, "files": 0}
        if _is_rank0():
            tau = self._tau()
            retained = {m: [v for v in ckpt.versions_needed_after(latest, tau.get(m, 0))] for m, latest in self.latest.items()}
            ckpt.write_weight_versions(path, step=step, latest=self.latest, retained=retained, tau=tau)
            if saver is None or info.get("workers"):
                ckpt.register_checkpoint(out, name=name, kind=kind, step=step, workers=info.get("workers", ()),
                                         extra={"metadata_only": True} if saver is None else None)
                ckpt.prune_checkpoints(out, self.run.checkpoints.keep_last_interval_steps)
        _rank_barrier()
        self.saved_steps.append(step)
        if self.trace is not None:
            self.trace.emit("runtime.checkpoint.save", "finish", step=step,
                            counters={"name": name, "kind": kind, "checkpoint_bytes": info.get("bytes", 0),
                                      "checkpoint_files": info.get("files", 0)})

    def on_node_complete(self, node, context, result):
        inner_hook = getattr(self.inner, "on_node_complete", None)
        if inner_hook is not None:
            inner_hook(node, context, result)
        pw = (result.counters or {}).get("produced_weight")
        if pw:
            self.latest[pw["model"]] = max(self.latest.get(pw["model"], 0), int(pw["version"]))
        closed = self.tracker.node_done(node)
        if closed is None:
            return
        iv = self.run.checkpoints.interval_steps
        if iv > 0 and closed % iv == 0 and closed < self.run.training.max_steps:
            self.save(closed, "interval")
            m = self.run.monitoring
            if m.test_inject_failure_after_checkpoint_step == closed and m.test_inject_failure_attempt == self.attempt:
                raise InjectedFailure(f"injected failure after the checkpoint of step {closed} (attempt {self.attempt})")
        elif closed == self.run.training.max_steps and self.run.checkpoints.save_final:
            self.save(closed, "final")


def run_with_replay(compiled, graph: RuntimeGraph, make_handler: Callable[[int], Any], trace: Optional[RuntimeTraceWriter], *,
                    node_timeout_s: Optional[float] = None, max_concurrency: Optional[int] = None) -> Dict[str, Any]:
    """Execute ``graph`` with up to ``monitoring.graph_replay_retries`` replays. ``make_handler(attempt)``
    builds a fresh handler per attempt; a handler may offer ``restore_checkpoint(entry, path)``."""
    run = compiled.run_config
    retries = int(run.monitoring.graph_replay_retries)
    out_dir = run.resolve(run.checkpoints.output_dir)
    current, restored_step, latest = graph, 0, {}
    completed_before: Set[str] = set()
    last_error: Optional[Exception] = None
    restore_path = None                     # directory of the verified entry the next attempt restores from
    if run.checkpoints.resume_from:
        src0 = run.resolve(run.checkpoints.resume_from)
        entry = ckpt.latest_usable_checkpoint(src0, verify_hashes=True)
        if entry is None:
            raise RuntimeExecutionError(f"checkpoints.resume_from={run.checkpoints.resume_from} holds no usable checkpoint")
        restored_step = int(entry["step"])
        restore_path = ckpt.entry_path(src0, entry)
        latest = dict(ckpt.read_weight_versions(restore_path)["latest"])
        current = suffix_graph(graph, restored_step)
        completed_before = set(graph.nodes) - set(current.nodes)
    for attempt in range(retries + 1):
        handler = make_handler(attempt)
        if hasattr(handler, "latest"):
            handler.latest.update(latest)
        hook = CheckpointingHook(handler, current, run, trace, attempt, latest)
        if (attempt > 0 or run.checkpoints.resume_from) and restored_step > 0:
            restore = getattr(handler, "restore_checkpoint", None)
            src = run.resolve(run.checkpoints.resume_from) if (attempt == 0 and run.checkpoints.resume_from) else out_dir
            if trace is not None:
                trace.emit("runtime.checkpoint.restore", "start", step=restored_step, counters={"attempt": attempt})
            if restore is not None:
                restore(restored_step, restore_path if restore_path is not None else
                        src / (f"step_{restored_step}" if (src / f"step_{restored_step}").exists() else "final"))
            if trace is not None:
                trace.emit("runtime.checkpoint.restore", "finish", step=restored_step, counters={"attempt": attempt})
        ex = RuntimeExecutor(current, run_id=run.run_id, handler=hook, trace=trace, node_timeout_s=node_timeout_s,
                             max_concurrency=max_concurrency)
        try:
            ctx = ex.run()
            return {"context": ctx, "attempts": attempt + 1, "restored_step": restored_step, "graph": current,
                    "completed_before": completed_before, "saved_steps": hook.saved_steps, "latest_versions": dict(hook.latest)}
        except RuntimeExecutionError as exc:
            last_error = exc
            if attempt == retries:
                break
            if trace is not None:
                trace.emit("runtime.graph", "replay", status="error", counters={"attempt": attempt + 1, "reason": str(exc)[:300]})
            entry = ckpt.latest_usable_checkpoint(out_dir, verify_hashes=True)
            if entry is not None and entry["kind"] == "interval":
                restored_step = int(entry["step"])
                restore_path = ckpt.entry_path(out_dir, entry)
                latest = dict(ckpt.read_weight_versions(restore_path)["latest"])
                current = suffix_graph(graph, restored_step)
            else:
                restored_step, latest, current, restore_path = 0, {}, graph, None
            completed_before = set(graph.nodes) - set(current.nodes)
            if trace is not None:
                trace.emit("runtime.graph", "recover", counters={"attempt": attempt + 1, "restored_step": restored_step,
                                                                 "skipped_nodes": len(completed_before),
                                                                 "suffix_nodes": len(current.nodes), "weight_versions": latest})
    raise RuntimeExecutionError(f"graph execution failed after {retries + 1} attempt(s): {last_error}") from last_error


def _is_rank0() -> bool:
    """True in the one process of a job that owns the checkpoint index (rank 0, or a job without ranks)."""
    try:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            return dist.get_rank() == 0
    except ImportError:
        pass
    import os
    return int(os.environ.get("RANK", "0")) == 0


def _rank_barrier() -> None:
    """All ranks leave a checkpoint together, after rank 0 has registered it and pruned the old ones."""
    try:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.barrier()
    except ImportError:
        pass
