"""Asynchronous dependency- and resource-driven executor of a ``RuntimeGraph``.

A node is launched when all its dependencies have completed and none of its resource keys is held;
among ready nodes the order is (logical step, transfers before operators, position in the graph's
order). Handlers give the nodes meaning: ``MetadataOnlyOperationHandler`` moves no tensors and
only produces the counters and version bookkeeping the trace verifier checks (the fake backend used
for CPU testing and replay tests); the engine handler runs the kernels. A handler may merge several
ready nodes into one launch (``select_batch`` / ``execute_batch``), which is how the fused
actor/critic training pair runs. Reference: RPEG/runtime/executor.py:25-469.
"""
from __future__ import annotations

import asyncio
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Set, Tuple

from ..passes.lower import ExecNodeType
from .containers import ContainerRef, ContainerStore, WeightVersion
from .errors import RuntimeExecutionError
from .graph import RuntimeGraph, RuntimeNodeSpec
from .trace import RuntimeTraceWriter
from .weight_versions import consumer_weight_version, uses_shadow_copies

TRAINABLE_NAMES = ("actor", "critic", "ac_share")
_MODEL_VALUE_TO_NAME = {"Pi": "actor", "V": "critic", "Ref": "reference", "R": "reward", "AC": "ac_share"}


@dataclass
class NodeExecutionResult:
    node_id: str
    status: str = "ok"
    counters: Dict[str, Any] = field(default_factory=dict)
    containers: Tuple[ContainerRef, ...] = ()
    weights: Tuple[WeightVersion, ...] = ()


@dataclass
class RuntimeExecutionContext:
    run_id: str
    store: ContainerStore
    completed: Dict[str, NodeExecutionResult] = field(default_factory=dict)
    logical_step: Optional[int] = None
    state: Dict[str, Any] = field(default_factory=dict)


def node_step(node: RuntimeNodeSpec) -> Optional[int]:
    return None if node.logical_step is None else int(node.logical_step)


def split_part_index(node_id: str) -> Optional[int]:
    for marker in (":g", ":i"):
        if marker in node_id:
            try:
                return int(node_id.rsplit(marker, 1)[1])
            except ValueError:
                return None
    return None


def model_name(model: Optional[str]) -> Optional[str]:
    return _MODEL_VALUE_TO_NAME.get(model, model) if model is not None else None


class MetadataOnlyOperationHandler:
    """Executes every node with references and counters only (no tensors, no GPU)."""

    def __init__(self, compiled: Any = None, fail_on: Optional[Dict[str, int]] = None):
        self.compiled = compiled
        self.fail_on = dict(fail_on or {})          # node-id substring -> number of times to fail (host-side injection)
        self.latest: Dict[str, int] = {}

    def tau_of(self, model: Optional[str]) -> int:
        if self.compiled is None or model is None:
            return 0
        for m, t in self.compiled.config.rpeg.tau.items():
            if _MODEL_VALUE_TO_NAME.get(m.value) == model_name(model):
                return int(t)
        return 0

    def quantile_counters(self, node: RuntimeNodeSpec) -> Dict[str, Any]:
        n = node.exec_node
        if n.n_seqs is None:
            return {}
        out: Dict[str, Any] = {"partial_n_seqs": int(n.n_seqs), "partial_is_prefill_phase": bool(n.is_prefill_phase)}
        if n.n_active is not None:
            out["partial_n_active"] = int(n.n_active)
        if n.phase_steps is not None:
            out["partial_phase_steps"] = int(n.phase_steps)
        if n.phase_t_start is not None:
            out["partial_phase_t_start"] = int(n.phase_t_start)
        part = split_part_index(node.node_id)
        if part is not None and self.compiled is not None:
            wl = self.compiled.workload
            q = wl.gen_quantiles or ()
            total = wl.B * wl.K
            out["artifact_part"], out["artifact_parts"] = part, len(q)
            out["partial_batch_offset"] = round(q[part - 1][0] * total) if part > 0 else 0
            if node.vertex_id in ("g_pi", "g_ac"):
                out["generation_length"] = int(q[part][1]) if q else wl.T
        return out

    async def execute(self, node: RuntimeNodeSpec, context: RuntimeExecutionContext) -> NodeExecutionResult:
        await asyncio.sleep(0)
        for needle, left in list(self.fail_on.items()):
            if needle in node.node_id and left > 0:
                self.fail_on[needle] = left - 1
                raise RuntimeError(f"injected failure at {node.node_id}")
        c: Dict[str, Any] = {"kind": node.kind.value, "dependency_count": len(node.dependencies),
                             "resource_count": len(node.resource_keys)}
        containers: List[ContainerRef] = []
        weights: List[WeightVersion] = []
        step = node_step(node)
        name = model_name(node.model)
        if node.kind is ExecNodeType.OP:
            c.update(self.quantile_counters(node))
            if name in TRAINABLE_NAMES and node.role in ("GEN", "INF") and step is not None:
                tau = self.tau_of(node.model)
                c.update(weight_version=consumer_weight_version(step, tau), model=name, shadow=uses_shadow_copies(tau))
            ref = ContainerRef(f"{node.node_id}:output", step or 0, split_part_index(node.node_id), producer=node.node_id)
            context.store.put(ref)
            containers.append(ref)
            if node.role == "TRAIN" and name is not None:
                version = self.latest.get(name, 0) + 1
                self.latest[name] = version
                shadow = uses_shadow_copies(self.tau_of(node.model))
                c["produced_weight"] = {"model": name, "version": version, "shadow": shadow}
                weights.append(WeightVersion(name, version, tuple(node.parallelism or (1, 1, 1))))
        else:
            c["payload_in_bytes"] = node.payload_in_bytes
            c["label"] = node.label
            ref = ContainerRef(f"{node.node_id}:{node.label or node.kind.value}", step or 0, None, nbytes=node.payload_in_bytes,
                               producer=node.node_id)
            context.store.put(ref)
            containers.append(ref)
        return NodeExecutionResult(node.node_id, "ok", c, tuple(containers), tuple(weights))


class RuntimeExecutor:
    def __init__(self, graph: RuntimeGraph, *, run_id: str, handler=None, trace: Optional[RuntimeTraceWriter] = None,
                 store: Optional[ContainerStore] = None, max_concurrency: Optional[int] = None,
                 node_timeout_s: Optional[float] = None, logical_step: Optional[int] = None):
        self.graph = graph
        self.run_id = run_id
        self.handler = handler or MetadataOnlyOperationHandler()
        self.trace = trace
        self.store = store or ContainerStore()
        self.max_concurrency = max_concurrency
        self.node_timeout_s = node_timeout_s
        self.logical_step = logical_step
        self._pos = {nid: i for i, nid in enumerate(graph.topological_order)}

    def run(self) -> RuntimeExecutionContext:
        return asyncio.run(self.run_async())

    def _step_of(self, node: RuntimeNodeSpec) -> Optional[int]:
        return self.logical_step if self.logical_step is not None else node_step(node)

    def _ready(self, pending: Set[str], done: Dict[str, NodeExecutionResult]) -> List[RuntimeNodeSpec]:
        ready = [self.graph.nodes[i] for i in self.graph.topological_order
                 if i in pending and all(d in done for d in self.graph.nodes[i].dependencies)]
        ready.sort(key=lambda n: (n.logical_step if n.logical_step is not None else 1 << 60,
                                  0 if n.kind is not ExecNodeType.OP else 1, self._pos[n.node_id]))
        return ready

    def _batch(self, node, ready, pending, occupied, context) -> Tuple[RuntimeNodeSpec, ...]:
        select = getattr(self.handler, "select_batch", None)
        if select is None:
            return (node,)
        picked = tuple(select(node, tuple(n for n in ready if n.node_id in pending), context) or (node,))
        if node not in picked:
            picked = (node, *picked)
        return picked

    async def _execute(self, nodes: Tuple[RuntimeNodeSpec, ...], context) -> Tuple[NodeExecutionResult, ...]:
        if len(nodes) > 1:
            return tuple(await self.handler.execute_batch(nodes, context))
        return (await self.handler.execute(nodes[0], context),)

    async def run_async(self) -> RuntimeExecutionContext:
        pending = set(self.graph.nodes)
        running: Dict[asyncio.Task, Tuple[RuntimeNodeSpec, ...]] = {}
        started: Dict[asyncio.Task, float] = {}
        done: Dict[str, NodeExecutionResult] = {}
        occupied: Set[str] = set()
        ctx = RuntimeExecutionContext(self.run_id, self.store, done, self.logical_step)
        while pending or running:
            launched = False
            ready = self._ready(pending, done)
            for node in ready:
                if node.node_id not in pending:
                    continue
                if self.max_concurrency is not None and len(running) >= self.max_concurrency:
                    break
                if occupied.intersection(node.resource_keys):
                    continue
                batch = self._batch(node, ready, pending, occupied, ctx)
                res: Set[str] = set()
                for b in batch:
                    res.update(b.resource_keys)
                if res & occupied:
                    continue
                for b in batch:
                    pending.discard(b.node_id)
                    if self.trace is not None:
                        info = {"kind": b.kind.value, "resources": list(b.resource_keys), "scheduled_at": time.time(),
                                "batch_scheduled_nodes": [x.node_id for x in batch]}
                        for k, v in (("model", model_name(b.model)), ("role", b.role), ("vertex_id", b.vertex_id),
                                     ("parallelism", b.parallelism), ("microbatch", b.microbatch), ("label", b.label)):
                            if v is not None:
                                info[k] = v
                        self.trace.emit(b.node_id, "start", worker_id=b.worker_id, step=self._step_of(b), counters=info)
                occupied |= res
                task = asyncio.create_task(self._execute(batch, ctx))
                running[task] = batch
                started[task] = time.perf_counter()
                launched = True
            if running:
                finished, _ = await asyncio.wait(running.keys(), timeout=self.node_timeout_s, return_when=asyncio.FIRST_COMPLETED)
                if not finished:
                    active = [n.node_id for t in running for n in running[t]]
                    for t in running:
                        t.cancel()
                    raise RuntimeExecutionError(f"runtime node timeout after {self.node_timeout_s:.1f}s; running nodes={active}")
                for task in finished:
                    nodes = running.pop(task)
                    dur = time.perf_counter() - started.pop(task)
                    for n in nodes:
                        occupied.difference_update(n.resource_keys)
                    try:
                        results = task.result()
                    except Exception as exc:
                        if self.trace is not None:
                            for n in nodes:
                                self.trace.emit(n.node_id, "finish", status="error", worker_id=n.worker_id, step=self._step_of(n),
                                                counters={"kind": n.kind.value, "duration_s": dur}, message=str(exc))
                        for t in running:
                            t.cancel()
                        raise RuntimeExecutionError(f"runtime node(s) {[n.node_id for n in nodes]} failed: {exc}") from exc
                    by_id = {r.node_id: r for r in results}
                    lost = [n.node_id for n in nodes if n.node_id not in by_id]
                    if lost:
                        raise RuntimeExecutionError(f"handler returned no result for nodes {lost}")
                    for n in nodes:
                        r = by_id[n.node_id]
                        r.counters.setdefault("duration_s", dur)
                        done[n.node_id] = r
                        if self.trace is not None:
                            self.trace.emit(n.node_id, "finish", status=r.status, worker_id=n.worker_id, step=self._step_of(n),
                                            counters=r.counters)
                        hook = getattr(self.handler, "on_node_complete", None)
                        if hook is not None:
                            out = hook(n, ctx, r)
                            if asyncio.iscoroutine(out):
                                await out
                continue
            if pending and not launched:
                blocked = {n.node_id: sorted(occupied.intersection(n.resource_keys)) for n in self._ready(pending, done)}
                if blocked:
                    raise RuntimeExecutionError(f"ready nodes are blocked with no running work: {blocked}")
                waiting = {i: sorted(set(self.graph.nodes[i].dependencies) - set(done)) for i in sorted(pending)}
                raise RuntimeExecutionError(f"runtime graph made no progress; unresolved dependencies: {waiting}")
        return ctx
