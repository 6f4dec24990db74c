"""Critical-path list scheduler over an executable graph (policy ``rpeg_critical_path_list_v1``).

Semantics reproduced from the reference (RPEG/schedule/scheduler.py:270-552):
  * node duration = ``cost_model.time(node)``; rank = duration + max rank of the successors; all
    quantile sub-nodes ``v@k:g*`` / ``v@k:i*`` of one chain share the chain's largest rank;
  * a node may start when its predecessors have finished and every device it reserves is free;
    COMM/RESHARD nodes reserve what the transfer-resource policy says (destination only by default);
  * ready nodes are taken in order of (earliest start, transfers before operators, template
    vertex index, higher rank first, insertion order), re-evaluating the earliest start on pop;
  * a fused ``t_pi``/``t_V`` pair is placed atomically with the makespan of the fused bidirectional
    pipeline schedule when both are ready (the first to become ready is parked until its peer is).

Implementation note: nodes and devices are mapped to dense integers once, and the inner loop works
on lists, which keeps one evaluation of a 32-GPU plan well under a millisecond-scale budget per
node for the simulated-annealing search.
"""
from __future__ import annotations

import heapq
import re
from typing import Dict, List, Optional, Sequence, Tuple

from ..analytic.cost import NodeCostModel
from ..core.types import DeviceSpace, RPEG_TRANSFER_RESOURCE_POLICY, TransferResourcePolicy
from ..passes.lower import ExecNode, ExecNodeType, ExecutableRPEG
from ..passes.transfer_resources import reserved_allocations
from .trace import Trace

_SUB = re.compile(r"^(.+@\d+):[gi](\d+)$")
POLICY_NAME = "rpeg_critical_path_list_v1"


def compute_ranks(executable: ExecutableRPEG, durations: Dict[ExecNode, float]) -> Dict[ExecNode, float]:
    succ: Dict[ExecNode, List[ExecNode]] = {n: [] for n in executable.nodes}
    indeg = {n: 0 for n in executable.nodes}
    for e in executable.edges:
        succ[e.src].append(e.dst)
        indeg[e.dst] += 1
    order, queue = [], [n for n in executable.nodes if indeg[n] == 0]
    head = 0
    while head < len(queue):
        u = queue[head]
        head += 1
        order.append(u)
        for w in succ[u]:
            indeg[w] -= 1
            if indeg[w] == 0:
                queue.append(w)
    rank: Dict[ExecNode, float] = {}
    for v in reversed(order):
        rank[v] = durations[v] + max((rank[w] for w in succ[v]), default=0.0)
    return rank


def fused_pipeline_duration(members: Sequence[ExecNode], durations: Dict[ExecNode, float]) -> float:
    """Makespan of actor and critic training run as one bidirectional pipeline; falls back to the
    serial sum when the pair cannot be fused (reference: scheduler.py:199-263)."""
    serial = sum(durations[m] for m in members)
    by_v = {m.template_id: m for m in members if m.op is not None}
    if set(by_v) != {"t_pi", "t_V"}:
        return serial
    actor, critic = by_v["t_pi"], by_v["t_V"]
    if actor.pi is None or actor.mb is None or critic.pi != actor.pi or critic.mb != actor.mb:
        return serial
    pp, mb = int(actor.pi[1]), int(actor.mb)
    slots = mb + pp - 1
    if pp <= 1 or mb < pp or slots <= 0:
        return serial
    from ..runtime.fused_pipeline import FusedPipelineModel, build_fused_pipeline_schedule

    def mk(name, node, reverse):
        fwd = float(durations[node]) / (3.0 * slots)
        return FusedPipelineModel.uniform(name, pipeline_stages=pp, microbatches=mb, forward_s=fwd,
                                          backward_s=2.0 * fwd, activation_bytes=0, reverse=reverse)

    return float(build_fused_pipeline_schedule((mk("actor", actor, False), mk("critic", critic, True))).makespan_s)


def schedule(executable: ExecutableRPEG, cost_model: NodeCostModel, device_space: DeviceSpace, *,
             transfer_resource_policy: TransferResourcePolicy = RPEG_TRANSFER_RESOURCE_POLICY,
             durations: Optional[Dict[ExecNode, float]] = None) -> Trace:
    nodes = executable.nodes
    n = len(nodes)
    index = {v: i for i, v in enumerate(nodes)}
    succ: List[List[int]] = [[] for _ in range(n)]
    indeg = [0] * n
    pred_ids = {v.id: set() for v in nodes}
    succ_ids = {v.id: set() for v in nodes}
    for e in executable.edges:
        a, b = index[e.src], index[e.dst]
        succ[a].append(b)
        indeg[b] += 1
        pred_ids[e.dst.id].add(e.src.id)
        succ_ids[e.src.id].add(e.dst.id)
    by_id = {v.id: v for v in nodes}
    reserved = {v: reserved_allocations(v, policy=transfer_resource_policy, predecessors=pred_ids,
                                        successors=succ_ids, by_id=by_id) for v in nodes}
    dev_cache: Dict[tuple, Tuple[int, ...]] = {}

    def devices(allocs) -> Tuple[int, ...]:
        out = set()
        for a in allocs:
            key = (a.origin, a.extent)
            if key not in dev_cache:
                dev_cache[key] = tuple(device_space.device_id(*c) for c in a.coords())
            out.update(dev_cache[key])
        return tuple(out)

    blocked = [devices(reserved[v]) for v in nodes]
    dur_map = durations if durations is not None else {v: cost_model.time(v) for v in nodes}
    dur = [dur_map[v] for v in nodes]
    rank_map = compute_ranks(executable, dur_map)
    chains: Dict[str, List[ExecNode]] = {}
    for v in nodes:
        m = _SUB.match(v.id)
        if m:
            chains.setdefault(m.group(1), []).append(v)
    for members in chains.values():
        top = max(rank_map[v] for v in members)
        for v in members:
            rank_map[v] = top
    rank = [rank_map[v] for v in nodes]
    templates = sorted({v.template_id for v in nodes if v.kind is ExecNodeType.OP and v.op is not None})
    t_order = {t: i for i, t in enumerate(templates)}
    topo = [t_order.get(v.template_id, 0) if (v.kind is ExecNodeType.OP and v.op is not None) else len(t_order) for v in nodes]
    prio = [1 if v.kind is ExecNodeType.OP else 0 for v in nodes]

    avail = [0.0] * device_space.num_devices()
    pred_done = [0.0] * n
    start = [None] * n
    finish = [None] * n
    ready = [False] * n
    parked: Dict[str, int] = {}
    placed: List[int] = []
    heap: list = []
    tie = 0

    def est(i: int) -> float:
        t = pred_done[i]
        for d in blocked[i]:
            if avail[d] > t:
                t = avail[d]
        return t

    def push(i: int) -> None:
        nonlocal tie
        heapq.heappush(heap, (est(i), prio[i], topo[i], -rank[i], tie, i))
        tie += 1
        ready[i] = True

    def release(i: int, t_fin: float) -> None:
        for w in succ[i]:
            indeg[w] -= 1
            if t_fin > pred_done[w]:
                pred_done[w] = t_fin
            if indeg[w] == 0:
                push(w)
                g = nodes[w].fusion_group
                if g and g in parked:
                    push(parked.pop(g))

    for i in range(n):
        if indeg[i] == 0:
            push(i)
    group_members: Dict[str, List[int]] = {}
    for i, v in enumerate(nodes):
        if v.fusion_group:
            group_members.setdefault(v.fusion_group, []).append(i)

    while heap:
        t_h, cp, ti, nr, _, i = heapq.heappop(heap)
        if not ready[i]:
            continue
        t_now = est(i)
        if t_now > t_h:
            heapq.heappush(heap, (t_now, cp, ti, nr, tie, i))
            tie += 1
            continue
        group = nodes[i].fusion_group
        pair = [i]
        if group is not None:
            pair = sorted((j for j in group_members[group] if ready[j]), key=lambda j: nodes[j].id)
            if len(pair) != 2:
                expected = group_members[group]
                if len(expected) == 2 and all(start[j] is None for j in expected):
                    ready[i] = False
                    parked[group] = i
                    continue
                pair = [i]
        if len(pair) == 2:
            t_grp = max(est(j) for j in pair)
            if t_grp > t_h:
                heapq.heappush(heap, (t_grp, cp, ti, nr, tie, i))
                tie += 1
                continue
            t_fin = t_grp + fused_pipeline_duration([nodes[j] for j in pair], dur_map)
            for j in pair:
                ready[j] = False
                start[j], finish[j] = t_grp, t_fin
                placed.append(j)
            for j in pair:
                for d in blocked[j]:
                    avail[d] = t_fin
            for j in pair:
                release(j, t_fin)
            continue
        ready[i] = False
        start[i], finish[i] = t_now, t_now + dur[i]
        placed.append(i)
        for d in blocked[i]:
            avail[d] = finish[i]
        release(i, finish[i])

    if any(s is None for s in start):
        missing = [nodes[i].id for i in range(n) if start[i] is None]
        raise ValueError(f"cycle in executable graph; unscheduled: {missing}")
    return Trace({v: start[i] for i, v in enumerate(nodes)}, {v: finish[i] for i, v in enumerate(nodes)}, reserved,
                 tuple(nodes[i] for i in placed))
