"""Lower an unrolled RPEG plus an execution plan into the executable graph the scheduler and the
runtime consume: OP nodes (one per vertex and iteration, split into quantile phases where that
lets inference overlap generation), COMM nodes for data crossing allocations, RESHARD nodes for a
layout change of a trainable model on the same devices, and ordering edges.

Rules reproduced from the reference's RPEG/passes/lower.py:330-851 (ids and counters included so
plans, traces and verifier output stay comparable):

1. OP nodes ``v@k``. With generation quantiles, a generation vertex that feeds at least one
   inference vertex on disjoint devices becomes chained phases ``v@k:g0 -> g1 -> ...``.
2. Data edges: same allocation -> plain edge, else ``comm{n}``. A split generation feeding a
   disjoint inference vertex splits that vertex into ``v@k:i0 ...`` and connects phase to phase with
   payload ``max(1, floor(payload * n_seqs_q / (B K)))``; otherwise only the last phase feeds on.
3. ``t_pi`` and ``t_V`` of one step are tagged ``actor_critic_train@k`` when fusion is on and they
   agree on allocation, parallelism, microbatches, ``pp > 1`` and ``mb >= pp``.
4. Consecutive vertices of the same trainable model inside a step: same devices but different
   parallelism -> ``reshard{n}`` between them; different devices -> ordering edge; shadow pairs
   (stale weights on disjoint devices) and data-reachable pairs on different devices are skipped.
5. Publication edges: identical layout -> edge; same devices -> RESHARD; else COMM whose payload is
   scaled by the share of devices that do not already hold the weights.
6. A reshard that returns a model to training is ordered before a reshard that publishes another
   model to serving on overlapping devices when the consumer depends on the producer's data.
7. One composite operator ``t_pi||V@k`` per fusion group.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from enum import Enum
from typing import Dict, List, Optional, Tuple

from ..analytic.models import ModelSuite
from ..analytic.workload import Workload
from ..core.types import Allocation, Model, Role, TemplateVertex
from ..ir.plan import ExecutionPlan
from ..ir.rpeg import RPEG
from .unroll import UnrolledNode, UnrolledRPEG


class ExecNodeType(Enum):
    OP = "op"
    COMM = "comm"
    RESHARD = "reshard"


@dataclass(frozen=True, eq=False)
class ExecNode:
    id: str
    kind: ExecNodeType
    allocs: Tuple[Allocation, ...]
    op: Optional[UnrolledNode] = None
    model: Optional[Model] = None
    pi: Optional[Tuple[int, int, int]] = None
    mb: Optional[int] = None
    n_seqs: Optional[int] = None
    n_active: Optional[int] = None
    phase_steps: Optional[int] = None
    phase_t_start: Optional[int] = None
    is_prefill_phase: bool = False
    fusion_group: Optional[str] = None
    payload_in_bytes: int = 0
    label: Optional[str] = None

    def __hash__(self) -> int:
        return hash(self.id)

    def __eq__(self, other) -> bool:
        return isinstance(other, ExecNode) and other.id == self.id

    @property
    def role(self) -> Optional[Role]:
        return None if self.op is None else self.op.template_vertex.kind.role

    @property
    def template_id(self) -> Optional[str]:
        return None if self.op is None else self.op.template_vertex.id


@dataclass(frozen=True)
class ExecEdge:
    src: ExecNode
    dst: ExecNode


@dataclass(frozen=True)
class CompositeExecOperator:
    id: str
    member_ids: Tuple[str, ...]
    invoked_models: Tuple[Model, ...]
    allocation: Allocation
    parallelism: Tuple[int, int, int]
    microbatch: int
    incoming: Tuple[str, ...]
    outgoing: Tuple[str, ...]


@dataclass(frozen=True)
class ExecutableRPEG:
    nodes: Tuple[ExecNode, ...]
    edges: Tuple[ExecEdge, ...]
    composite_operators: Tuple[CompositeExecOperator, ...] = ()

    def by_id(self) -> Dict[str, ExecNode]:
        return {n.id: n for n in self.nodes}


def node_id(x: UnrolledNode) -> str:
    return x.id


def allocs_disjoint(a: Allocation, b: Allocation) -> bool:
    return not a.overlaps(b)


@dataclass(frozen=True)
class GenPhase:
    n_active: int      # rows still generating when the phase starts
    n_seqs: int        # rows that finish inside the phase
    steps: int         # decode steps of the phase
    t_start: int       # decode step index at which the phase starts
    is_prefill: bool


def generation_phases(workload: Workload) -> List[GenPhase]:
    """Quantile ``(f, t)``: ``round(f*B*K)`` rows are done after ``t`` tokens; prefill yields the
    first token, so ``t`` tokens need ``t-1`` decode steps."""
    total = workload.B * workload.K
    phases, prev_step, prev_done = [], 0, 0
    for q, (frac, tokens) in enumerate(workload.gen_quantiles or ()):
        done = round(frac * total)
        step = tokens - 1
        phases.append(GenPhase(total - prev_done, done - prev_done, max(0, step - prev_step), prev_step, q == 0))
        prev_step, prev_done = step, done
    return phases


def data_reachable(rpeg: RPEG) -> set:
    succ: Dict[str, List[str]] = {v.id: [] for v in rpeg.vertices}
    for e in rpeg.data_edges:
        succ[e.src.id].append(e.dst.id)
    reach = set()
    for v in rpeg.vertices:
        stack, seen = list(succ[v.id]), set()
        while stack:
            w = stack.pop()
            if w not in seen:
                seen.add(w)
                reach.add((v.id, w))
                stack.extend(succ[w])
    return reach


def within_step_priors(order: Tuple[TemplateVertex, ...], trainable) -> List[Tuple[TemplateVertex, TemplateVertex, Model]]:
    last: Dict[Model, TemplateVertex] = {}
    pairs = []
    for v in order:
        m = v.kind.model
        if m in trainable:
            if m in last:
                pairs.append((last[m], v, m))
            last[m] = v
    return pairs


class _Builder:
    def __init__(self, rpeg, unrolled, plan, suite, workload, fusion):
        self.rpeg, self.unrolled, self.plan, self.suite, self.workload, self.fusion = rpeg, unrolled, plan, suite, workload, fusion
        self.nodes: Dict[str, ExecNode] = {}
        self.edges: List[Tuple[str, str]] = []
        self._edge_seen = set()
        self.comm_ctr = 0
        self.reshard_ctr = 0
        self.phases = generation_phases(workload) if (workload and workload.gen_quantiles) else []
        self.gen_subs: Dict[str, List[str]] = {}
        self.inf_subs: Dict[str, List[str]] = {}

    # -- helpers
    def sigma(self, v: TemplateVertex) -> Allocation:
        return self.plan.sigma[v.id]

    def edge(self, u: str, v: str) -> None:
        if (u, v) not in self._edge_seen:
            self._edge_seen.add((u, v))
            self.edges.append((u, v))

    def op_node(self, nid: str, x: UnrolledNode, **extra) -> ExecNode:
        v = x.template_vertex
        node = ExecNode(nid, ExecNodeType.OP, (self.sigma(v),), op=x, model=v.kind.model, pi=self.plan.pi[v.id],
                        mb=self.plan.mb.get(v.id), **extra)
        self.nodes[nid] = node
        return node

    def first(self, nid: str) -> str:
        return (self.gen_subs.get(nid) or self.inf_subs.get(nid) or [nid])[0]

    def last(self, nid: str) -> str:
        return (self.gen_subs.get(nid) or self.inf_subs.get(nid) or [nid])[-1]

    def link(self, u: str, v: str, payload: int, label: str) -> None:
        """Edge if both sit on the same allocation, else a COMM node in between."""
        a, b = self.nodes[u].allocs[0], self.nodes[v].allocs[0]
        if a == b:
            self.edge(u, v)
            return
        self.comm_ctr += 1
        c = ExecNode(f"comm{self.comm_ctr}", ExecNodeType.COMM, (a, b), payload_in_bytes=payload, label=label)
        self.nodes[c.id] = c
        self.edge(u, c.id)
        self.edge(c.id, v)

    def reshard(self, u: str, v: str, model: Model) -> None:
        self.reshard_ctr += 1
        payload = self.suite.n_params(model) * self.suite.specs[model].dtype_bytes
        r = ExecNode(f"reshard{self.reshard_ctr}", ExecNodeType.RESHARD,
                     (self.nodes[u].allocs[0], self.nodes[v].allocs[0]), model=model, payload_in_bytes=payload,
                     label=f"W_{model.value}")
        self.nodes[r.id] = r
        self.edge(u, r.id)
        self.edge(r.id, v)

    # -- steps
    def make_ops(self) -> None:
        split_gen = set()
        if self.phases:
            for e in self.unrolled.data_edges:
                s, d = e.src.template_vertex, e.dst.template_vertex
                if s.kind.role is Role.GENERATION and d.kind.role is Role.INFERENCE and allocs_disjoint(self.sigma(s), self.sigma(d)):
                    split_gen.add(s.id)
        for x in self.unrolled.nodes:
            v = x.template_vertex
            if v.kind.role is Role.GENERATION and v.id in split_gen:
                ids = []
                for q, ph in enumerate(self.phases):
                    sid = f"{v.id}@{x.k}:g{q}"
                    self.op_node(sid, x, n_seqs=ph.n_seqs, n_active=ph.n_active, phase_steps=ph.steps,
                                 phase_t_start=ph.t_start, is_prefill_phase=ph.is_prefill)
                    ids.append(sid)
                for a, b in zip(ids, ids[1:]):
                    self.edge(a, b)
                self.gen_subs[x.id] = ids
            else:
                self.op_node(x.id, x)

    def split_inference(self, x: UnrolledNode) -> None:
        v = x.template_vertex
        self.nodes.pop(x.id, None)
        ids = []
        for q, ph in enumerate(self.phases):
            sid = f"{v.id}@{x.k}:i{q}"
            self.op_node(sid, x, n_seqs=ph.n_seqs)
            ids.append(sid)
        for a, b in zip(ids, ids[1:]):
            self.edge(a, b)
        self.inf_subs[x.id] = ids

    def data_edges(self) -> None:
        def gen_to_inf(e):
            return e.src.id in self.gen_subs and e.dst.template_vertex.kind.role is Role.INFERENCE

        ordered = [e for e in self.unrolled.data_edges if gen_to_inf(e)] + \
                  [e for e in self.unrolled.data_edges if not gen_to_inf(e)]
        total = self.workload.B * self.workload.K if self.workload else 1
        for e in ordered:
            payload, label = e.container.bytes(), e.container.name
            if gen_to_inf(e):
                if allocs_disjoint(self.sigma(e.src.template_vertex), self.sigma(e.dst.template_vertex)):
                    if e.dst.id not in self.inf_subs:
                        self.split_inference(e.dst)
                    for q, ph in enumerate(self.phases):
                        part = max(1, int(payload * (ph.n_seqs / total)))
                        self.link(self.gen_subs[e.src.id][q], self.inf_subs[e.dst.id][q], part, label)
                else:
                    self.link(self.gen_subs[e.src.id][-1], e.dst.id, payload, label)
            elif e.src.id in self.gen_subs:
                self.link(self.gen_subs[e.src.id][-1], e.dst.id, payload, label)
            elif e.src.id in self.inf_subs:
                if e.dst.id not in self.nodes:
                    raise KeyError(f"destination node {e.dst.id} not found")
                self.link(self.inf_subs[e.src.id][-1], e.dst.id, payload, label)
            else:
                self.link(e.src.id, e.dst.id, payload, label)

    def annotate_fusion(self) -> None:
        if not self.fusion:
            return
        steps: Dict[int, Dict[str, str]] = {}
        for x in self.unrolled.nodes:
            if x.template_vertex.id in ("t_pi", "t_V"):
                steps.setdefault(x.k, {})[x.template_vertex.id] = x.id
        for k, pair in steps.items():
            if set(pair) != {"t_pi", "t_V"}:
                continue
            a, c = self.nodes[pair["t_pi"]], self.nodes[pair["t_V"]]
            if (a.allocs == c.allocs and a.pi == c.pi and a.mb == c.mb and a.pi is not None and a.pi[1] > 1
                    and int(a.mb or 1) >= a.pi[1]):
                group = f"actor_critic_train@{k}"
                self.nodes[a.id] = replace(a, fusion_group=group)
                self.nodes[c.id] = replace(c, fusion_group=group)

    def intra_step_reshards(self, K_eval: int) -> set:
        resharded = set()
        reach = data_reachable(self.rpeg)
        for u_t, v_t, model in within_step_priors(self.rpeg.topological_vertices(), self.rpeg.trainable):
            au, av = self.sigma(u_t), self.sigma(v_t)
            if self.rpeg.tau.get(model, 0) > 0 and allocs_disjoint(au, av):
                continue  # shadow copy: the serving side runs on published (stale) weights elsewhere
            if (u_t.id, v_t.id) in reach and au != av:
                continue
            for k in range(K_eval):
                u, v = self.last(f"{u_t.id}@{k}"), self.first(f"{v_t.id}@{k}")
                nu, nv = self.nodes[u], self.nodes[v]
                if nu.allocs[0] == nv.allocs[0] and nu.pi == nv.pi:
                    continue
                if nu.allocs[0] != nv.allocs[0]:
                    self.edge(u, v)
                else:
                    self.reshard(u, v, model)
                    resharded.add(v_t.id)
        return resharded

    def publication_edges(self, resharded: set) -> None:
        for e in self.unrolled.pub_edges:
            u, v = e.src.id, self.first(e.dst.id)
            nu, nv = self.nodes[u], self.nodes[v]
            if nv.op.template_vertex.id in resharded:
                continue
            if nu.allocs[0] == nv.allocs[0]:
                if nu.pi == nv.pi:
                    self.edge(u, v)
                else:
                    self.reshard(u, v, nu.model)
                continue
            full = self.suite.n_params(nu.model) * self.suite.specs[nu.model].dtype_bytes
            n_max = max(nu.allocs[0].size(), nv.allocs[0].size())
            overlap = nu.allocs[0].overlap_size(nv.allocs[0])
            payload = full * (n_max - overlap) // n_max if n_max > 0 else full
            self.comm_ctr += 1
            c = ExecNode(f"comm{self.comm_ctr}", ExecNodeType.COMM, (nu.allocs[0], nv.allocs[0]),
                         payload_in_bytes=payload, label=f"W_{nu.model.value}")
            self.nodes[c.id] = c
            self.edge(u, c.id)
            self.edge(c.id, v)

    def lifetime_barriers(self) -> None:
        preds: Dict[str, List[str]] = {}
        succs: Dict[str, List[str]] = {}
        for u, v in self.edges:
            preds.setdefault(v, []).append(u)
            succs.setdefault(u, []).append(v)
        reach = data_reachable(self.rpeg)
        returns, publishes = [], []
        for t in list(self.nodes.values()):
            if t.kind is not ExecNodeType.RESHARD:
                continue
            ps = [self.nodes[i] for i in preds.get(t.id, ()) if self.nodes[i].kind is ExecNodeType.OP]
            ss = [self.nodes[i] for i in succs.get(t.id, ()) if self.nodes[i].kind is ExecNodeType.OP]
            if len(ps) != 1 or len(ss) != 1:
                continue
            p, s = ps[0], ss[0]
            if p.model is not s.model or p.model not in self.rpeg.trainable:
                continue
            if p.role is not Role.TRAINING and s.role is Role.TRAINING:
                returns.append((t, p))
            elif p.role is Role.TRAINING and s.role is not Role.TRAINING:
                publishes.append((t, s))
        for rt, producer in returns:
            for pt, consumer in publishes:
                if producer.model is consumer.model or producer.op.k != consumer.op.k:
                    continue
                if allocs_disjoint(producer.allocs[0], consumer.allocs[0]):
                    continue
                if (producer.template_id, consumer.template_id) in reach:
                    self.edge(rt.id, pt.id)

    def composites(self, edges: Tuple[ExecEdge, ...]) -> Tuple[CompositeExecOperator, ...]:
        out = []
        for group in sorted({n.fusion_group for n in self.nodes.values() if n.fusion_group}):
            members = sorted((n for n in self.nodes.values() if n.fusion_group == group), key=lambda n: n.template_id or n.id)
            if len(members) != 2 or any(m.pi is None or m.mb is None for m in members):
                continue
            ids = {m.id for m in members}
            incoming = sorted({e.src.id for e in edges if e.dst.id in ids and e.src.id not in ids})
            outgoing = sorted({e.dst.id for e in edges if e.src.id in ids and e.dst.id not in ids})
            step = group.rsplit("@", 1)[-1]
            out.append(CompositeExecOperator(f"t_pi||V@{step}", tuple(m.id for m in members),
                                             tuple(m.model for m in members), members[0].allocs[0], members[0].pi,
                                             int(members[0].mb), tuple(incoming), tuple(outgoing)))
        return tuple(out)


def lower(rpeg: RPEG, unrolled: UnrolledRPEG, plan: ExecutionPlan, suite: ModelSuite, K_eval: int,
          workload: Optional[Workload] = None, intra_stage_fusion: bool = False, verbose: bool = False) -> ExecutableRPEG:
    b = _Builder(rpeg, unrolled, plan, suite, workload, intra_stage_fusion)
    b.make_ops()
    b.data_edges()
    b.annotate_fusion()
    resharded = b.intra_step_reshards(K_eval)
    b.publication_edges(resharded)
    b.lifetime_barriers()
    edges = tuple(ExecEdge(b.nodes[u], b.nodes[v]) for u, v in b.edges)
    lowered = ExecutableRPEG(tuple(b.nodes.values()), edges, b.composites(edges))
    if verbose:
        kinds = [n.kind for n in lowered.nodes]
        print(f"lowered: {len(kinds)} nodes ({kinds.count(ExecNodeType.OP)} op, {kinds.count(ExecNodeType.COMM)} comm, "
              f"{kinds.count(ExecNodeType.RESHARD)} reshard), {len(edges)} edges")
    return lowered
