"""Runtime graph: the lowered executable graph annotated with what the executor needs, i.e.
dependencies, the worker that owns each operator, the logical step, and the resource keys a node
holds while it runs (``gpu:r:n:g`` for devices, ``worker:<id>`` for a model instance).

Resource rules follow the reference (RPEG/runtime/graph.py:91-449): an OP holds its worker and all
GPUs of its allocation; a transfer holds the GPUs the transfer-resource policy reserves plus the
destination worker (destination-only) or both adjacent workers. Weight transfers that leave a
training node of a step that writes a checkpoint additionally wait for every training node of that
step, so a checkpoint always sees a consistent set of models.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import Any, Dict, Iterable, List, Optional, Sequence, Set, Tuple

from ..core.types import Allocation, TransferResourcePolicy
from ..passes.lower import ExecNode, ExecNodeType, ExecutableRPEG
from ..passes.transfer_resources import reserved_allocations, transfer_reserves_destination_only
from .errors import RuntimeConfigError


@dataclass(frozen=True)
class RuntimeNodeSpec:
    node_id: str
    kind: ExecNodeType
    exec_node: ExecNode
    dependencies: Tuple[str, ...]
    successors: Tuple[str, ...]
    worker_id: Optional[str]
    vertex_id: Optional[str]
    model: Optional[str]
    role: Optional[str]
    parallelism: Optional[Tuple[int, int, int]]
    microbatch: Optional[int]
    allocations: Tuple[Allocation, ...]
    resource_keys: Tuple[str, ...]
    payload_in_bytes: int = 0
    label: Optional[str] = None
    logical_step: Optional[int] = None
    source_vertex_id: Optional[str] = None
    destination_vertex_id: Optional[str] = None

    def to_summary(self) -> dict:
        return {"node_id": self.node_id, "kind": self.kind.value, "dependencies": list(self.dependencies),
                "successors": list(self.successors), "worker_id": self.worker_id, "vertex_id": self.vertex_id,
                "model": self.model, "role": self.role, "parallelism": self.parallelism, "microbatch": self.microbatch,
                "resource_keys": list(self.resource_keys), "payload_in_bytes": self.payload_in_bytes, "label": self.label,
                "logical_step": self.logical_step, "source_vertex_id": self.source_vertex_id,
                "destination_vertex_id": self.destination_vertex_id, "fusion_group": self.exec_node.fusion_group}


@dataclass(frozen=True)
class RuntimeGraph:
    nodes: Dict[str, RuntimeNodeSpec]
    topological_order: Tuple[str, ...]
    composite_operators: Tuple[dict, ...] = ()

    @property
    def edges(self) -> Tuple[Tuple[str, str], ...]:
        return tuple((s, d) for s, n in self.nodes.items() for d in n.successors)

    def summary(self) -> dict:
        counts: Dict[str, int] = {}
        for n in self.nodes.values():
            counts[n.kind.value] = counts.get(n.kind.value, 0) + 1
        return {"node_count": len(self.nodes), "edge_count": len(self.edges), "counts": counts,
                "topological_order": list(self.topological_order),
                "nodes": [self.nodes[i].to_summary() for i in self.topological_order],
                "composite_operators": list(self.composite_operators)}

    def subgraph(self, keep: Set[str]) -> "RuntimeGraph":
        """Graph restricted to ``keep`` (dependencies on dropped nodes are considered satisfied)."""
        nodes = {}
        for nid in self.topological_order:
            if nid not in keep:
                continue
            n = self.nodes[nid]
            nodes[nid] = RuntimeNodeSpec(**{**n.__dict__, "dependencies": tuple(d for d in n.dependencies if d in keep),
                                            "successors": tuple(s for s in n.successors if s in keep)})
        return RuntimeGraph(nodes, tuple(i for i in self.topological_order if i in keep), self.composite_operators)


def suffix_node_ids(graph: "RuntimeGraph", restored_step: int) -> Set[str]:
    """Nodes that run after the state at the end of logical step ``restored_step`` was restored: every
    node of a later step, plus the transfers that cross the boundary (a weight publication or an
    activation hand-over that leaves a covered step and feeds a later one must be sent again)."""
    keep = {nid for nid, n in graph.nodes.items() if n.logical_step is None or int(n.logical_step) > restored_step}
    for nid in reversed(graph.topological_order):
        n = graph.nodes[nid]
        if nid not in keep and n.kind is not ExecNodeType.OP and any(s in keep for s in n.successors):
            keep.add(nid)
    return keep


def gpu_keys(alloc: Allocation) -> Tuple[str, ...]:
    return tuple(f"gpu:{r}:{n}:{g}" for r, n, g in alloc.coords())


def unrolled_step(node_id: str) -> Optional[int]:
    at = node_id.rfind("@")
    if at < 0:
        return None
    try:
        return int(node_id[at + 1:].split(":", 1)[0].split(".", 1)[0])
    except ValueError:
        return None


def _logical_step(node: ExecNode, preds: Set[str], succs: Set[str]) -> Optional[int]:
    if node.op is not None:
        return int(node.op.k) + 1
    for adj in (*sorted(preds), *sorted(succs)):
        k = unrolled_step(adj)
        if k is not None:
            return k + 1
    return None


def _adjacent_vertex(ids: Iterable[str]) -> Optional[str]:
    for i in sorted(ids):
        if "@" in i:
            return i.split("@", 1)[0]
    return None


def _add_checkpoint_barriers(by_id, preds, succs, steps: Set[int]) -> None:
    if not steps:
        return
    train: Dict[int, Set[str]] = {}
    for nid, n in by_id.items():
        if n.kind is ExecNodeType.OP and n.op is not None and n.role is not None and n.role.value == "TRAIN":
            train.setdefault(int(n.op.k), set()).add(nid)
    for nid, n in by_id.items():
        if n.kind is ExecNodeType.OP or not str(n.label or "").startswith("W_"):
            continue
        src_steps = {unrolled_step(p) for p in preds[nid] if unrolled_step(p) is not None and p in train.get(unrolled_step(p), ())}
        for k in src_steps & steps:
            for t in train.get(k, ()):
                if t != nid:
                    preds[nid].add(t)
                    succs[t].add(nid)


def build_runtime_graph(lowered: ExecutableRPEG, workers: Sequence[Any], *, preferred_order: Optional[Sequence[str]] = None,
                        transfer_resource_policy: Optional[TransferResourcePolicy] = None,
                        checkpoint_barrier_steps: Iterable[int] = ()) -> RuntimeGraph:
    ids = [n.id for n in lowered.nodes]
    if len(set(ids)) != len(ids):
        raise RuntimeConfigError("lowered graph has duplicate node ids")
    policy = transfer_resource_policy or TransferResourcePolicy("both_endpoints", "both_endpoints")
    by_id = {n.id: n for n in lowered.nodes}
    preds: Dict[str, Set[str]] = {i: set() for i in ids}
    succs: Dict[str, Set[str]] = {i: set() for i in ids}
    for e in lowered.edges:
        if e.src.id not in by_id or e.dst.id not in by_id:
            raise RuntimeConfigError(f"edge references an unknown node: {e.src.id}->{e.dst.id}")
        succs[e.src.id].add(e.dst.id)
        preds[e.dst.id].add(e.src.id)
    _add_checkpoint_barriers(by_id, preds, succs, set(checkpoint_barrier_steps))
    if preferred_order is None:
        indeg = {i: len(preds[i]) for i in ids}
        ready = deque(sorted(i for i, d in indeg.items() if d == 0))
        order: List[str] = []
        while ready:
            i = ready.popleft()
            order.append(i)
            for s in sorted(succs[i]):
                indeg[s] -= 1
                if indeg[s] == 0:
                    ready.append(s)
        if len(order) != len(ids):
            raise RuntimeConfigError("lowered graph contains a dependency cycle")
    else:
        order = list(preferred_order)
        if len(set(order)) != len(order) or set(order) != set(ids):
            raise RuntimeConfigError("preferred runtime order does not cover the node set exactly once")
        pos = {i: k for k, i in enumerate(order)}
        for i, ds in preds.items():
            for d in ds:
                if pos[d] >= pos[i]:
                    raise RuntimeConfigError(f"preferred runtime order violates dependency {d}->{i}")
    worker_of = {vid: w for w in workers for vid in (getattr(w, "owned_vertex_ids", None) or (w.vertex_id,))}

    def worker_key_of(node_id: str) -> Optional[str]:
        n = by_id.get(node_id)
        if n is None or n.op is None:
            return None
        w = worker_of.get(n.op.template_vertex.id)
        return None if w is None else f"worker:{w.worker_id}"

    specs: Dict[str, RuntimeNodeSpec] = {}
    for nid in order:
        n = by_id[nid]
        worker = vertex = role = model = None
        if n.kind is ExecNodeType.OP:
            if n.op is None:
                raise RuntimeConfigError(f"OP node {nid} lacks its unrolled operator")
            vertex, role = n.op.template_vertex.id, n.op.template_vertex.kind.role.value
            worker = worker_of.get(vertex)
            if worker is None:
                raise RuntimeConfigError(f"OP node {nid} has no worker for vertex {vertex}")
            model = worker.model
        elif n.model is not None:
            model = n.model.value
        keys: Set[str] = set()
        if worker is not None:
            keys.add(f"worker:{worker.worker_id}")
        if n.kind is not ExecNodeType.OP and len(n.allocs) >= 2:
            if transfer_reserves_destination_only(n, policy=policy, predecessors=preds, successors=succs, by_id=by_id):
                for s in sorted(succs[nid]):
                    k = worker_key_of(s)
                    if k:
                        keys.add(k)
                        break
            else:
                for adj in (*sorted(preds[nid]), *sorted(succs[nid])):
                    k = worker_key_of(adj)
                    if k:
                        keys.add(k)
            for a in reserved_allocations(n, policy=policy, predecessors=preds, successors=succs, by_id=by_id):
                keys.update(gpu_keys(a))
        else:
            for a in n.allocs:
                keys.update(gpu_keys(a))
        is_transfer = n.kind is not ExecNodeType.OP
        specs[nid] = RuntimeNodeSpec(
            nid, n.kind, n, tuple(sorted(preds[nid])), tuple(sorted(succs[nid])), None if worker is None else worker.worker_id,
            vertex, model, role, n.pi, n.mb, n.allocs, tuple(sorted(keys)), n.payload_in_bytes, n.label,
            _logical_step(n, preds[nid], succs[nid]), _adjacent_vertex(preds[nid]) if is_transfer else None,
            _adjacent_vertex(succs[nid]) if is_transfer else None)
    composites = tuple({"operator_id": c.id, "member_node_ids": list(c.member_ids),
                        "invoked_models": [m.value for m in c.invoked_models],
                        "allocation": {"origin": list(c.allocation.origin), "extent": list(c.allocation.extent)},
                        "parallelism": list(c.parallelism), "microbatch": c.microbatch,
                        "incoming_dependencies": list(c.incoming), "outgoing_publications": list(c.outgoing),
                        "runtime_projection": "coordinated_bidirectional_microtasks"} for c in lowered.composite_operators)
    return RuntimeGraph(specs, tuple(order), composites)
