"""Neighbourhood of the plan search: valid parallel degrees, the per-vertex candidate directory,
the single-vertex move kernel and the donor/receiver pair kernel.

Rules kept from the reference (RPEG/search/moves.py:97-950): TP divides the GPUs of a node; PP is 1
or an even divisor of the layer count; DP divides the prompt batch and leaves at least 8 prompts
per replica when dp > 1; microbatch counts are 1 without pipelining, else divisors of the local
batch with ``pp <= mb`` and at least 8 prompts per microbatch; origins are multiples of the extent;
the directory keeps, per vertex, every memory-feasible (dp, pp, tp, rack extent, node extent, mb)
sorted by isolated run time (at most 1000); a move picks a vertex (60 % weighted by its time on the
critical chain), proposes one re-placement plus strategies from a temperature-scaled window around
the current position; a pair move shrinks a donor and re-samples an overlapping receiver.

All randomness goes through one ``random.Random`` owned by the caller, so a search is reproducible
from its seed regardless of what else uses the global generator.
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Set, Tuple

from ..analytic.cost import NodeCostModel
from ..analytic.memory import NodeMemoryModel
from ..analytic.models import ModelSuite
from ..analytic.workload import Workload
from ..core.types import Allocation, DeviceSpace, TemplateVertex, packing_geometry, rectangular_node_layouts
from ..ir.plan import ExecutionPlan
from ..ir.rpeg import RPEG
from ..passes.lower import ExecNode, ExecNodeType, ExecutableRPEG
from ..passes.unroll import UnrolledNode
from ..schedule.trace import Trace
from .evaluate import Configuration

MIN_B_LOCAL = 8
Strategy = Tuple[int, int, int, int, int, int]  # dp, pp, tp, rack extent, node extent, microbatches


@dataclass
class SearchFlags:
    """Ablation switches (A3 fixed microbatching, A6 uniform vertex choice)."""
    fixed_mb: bool = False
    uniform_vertex: bool = False


@dataclass
class MoveStats:
    n_calls: int = 0
    n_placement_proposed: int = 0
    n_strategy_proposed: int = 0
    n_fallback: int = 0
    n_empty: int = 0
    n_pair_proposed: int = 0
    n_pair_accepted: int = 0
    n_pair_failed: int = 0
    n_pair_rejected: int = 0

    def summary(self, accepted_strategy: int = 0, accepted_placement: int = 0, rejected: int = 0) -> str:
        sv = self.n_placement_proposed + self.n_strategy_proposed
        acc = accepted_strategy + accepted_placement + self.n_pair_accepted
        tot = acc + rejected + self.n_pair_rejected
        return (f"  single-vertex proposals {sv} (strategy {self.n_strategy_proposed}, placement {self.n_placement_proposed}, "
                f"empty {self.n_empty}); pair proposals {self.n_pair_proposed} (accepted {self.n_pair_accepted}, "
                f"failed {self.n_pair_failed}); accepted {acc}/{max(1, tot)} ({100.0 * acc / max(1, tot):.1f}%)")


def valid_tp_degrees(G: int) -> List[int]:
    return [t for t in range(1, G + 1) if G % t == 0]


def valid_pp_degrees(R: int, N: int, G: int, L: int) -> List[int]:
    return [p for p in range(1, R * N * G + 1) if L % p == 0 and (p == 1 or p % 2 == 0)]


def valid_dp_degrees(R: int, N: int, B: int, G: int = 1) -> List[int]:
    return [d for d in range(1, R * N * G + 1) if B % d == 0]


def valid_mb_counts(pp: int, dp: int, B: int, flags: Optional[SearchFlags] = None) -> List[int]:
    local = B // dp
    if local < MIN_B_LOCAL and dp > 1:
        return []
    if pp == 1:
        return [1]
    if flags is not None and flags.fixed_mb:
        return [pp] if local % pp == 0 else [1]
    hi = min(local // MIN_B_LOCAL, local)
    return [m for m in range(pp, hi + 1) if local % m == 0]


def aligned_origins(extent: Tuple[int, int, int], space: DeviceSpace, r_lo: int = 0, r_hi: Optional[int] = None):
    r_ext, n_ext, g_ext = extent
    r_hi = space.R if r_hi is None else r_hi
    return ([r_lo + i * r_ext for i in range((r_hi - r_lo) // r_ext)], [i * n_ext for i in range(space.N // n_ext)],
            [i * g_ext for i in range(space.G // g_ext)])


def sample_origin(rng: random.Random, extent, space: DeviceSpace, r_lo: int = 0, r_hi: Optional[int] = None):
    rs, ns, gs = aligned_origins(extent, space, r_lo, r_hi)
    if not rs or not ns or not gs:
        return None
    return (rng.choice(rs), rng.choice(ns), rng.choice(gs))


def sample_strategy(rng: random.Random, v: TemplateVertex, suite: ModelSuite, space: DeviceSpace, workload: Workload,
                    r_lo: int = 0, r_hi: Optional[int] = None, flags: Optional[SearchFlags] = None):
    """Random valid (allocation, (dp, pp, tp), mb) inside racks ``[r_lo, r_hi)``, or ``None``."""
    R, N, G, B = space.R, space.N, space.G, workload.B
    r_hi = R if r_hi is None else r_hi
    racks = r_hi - r_lo
    tp = rng.choice(valid_tp_degrees(G))
    pps = valid_pp_degrees(R, N, G, suite.specs[v.kind.model].L)
    if not pps:
        return None
    pp = rng.choice(pps)
    dps = [d for d in valid_dp_degrees(R, N, B, G)
           if (geom := packing_geometry(d, pp, tp, G)) is not None and geom[1] <= racks * N]
    if not dps:
        return None
    dp = rng.choice(dps)
    g_ext, nodes = packing_geometry(dp, pp, tp, G)
    layouts = rectangular_node_layouts(nodes, racks, N)
    if not layouts:
        return None
    r_ext, n_ext = rng.choice(layouts)
    origin = sample_origin(rng, (r_ext, n_ext, g_ext), space, r_lo, r_hi)
    mbs = valid_mb_counts(pp, dp, B, flags)
    if origin is None or not mbs:
        return None
    return Allocation(origin, (r_ext, n_ext, g_ext)), (dp, pp, tp), rng.choice(mbs)


def enumerate_strategies(v: TemplateVertex, suite: ModelSuite, space: DeviceSpace, workload: Workload,
                         flags: Optional[SearchFlags] = None) -> List[Strategy]:
    R, N, G, B = space.R, space.N, space.G, workload.B
    out: List[Strategy] = []
    for tp in valid_tp_degrees(G):
        for pp in valid_pp_degrees(R, N, G, suite.specs[v.kind.model].L):
            for dp in valid_dp_degrees(R, N, B, G):
                mbs = valid_mb_counts(pp, dp, B, flags)
                geom = packing_geometry(dp, pp, tp, G)
                if not mbs or geom is None:
                    continue
                for r_ext, n_ext in rectangular_node_layouts(geom[1], R, N):
                    out.extend((dp, pp, tp, r_ext, n_ext, mb) for mb in mbs)
    return out


def mock_node(v: TemplateVertex, strat: Strategy, g_ext: int) -> ExecNode:
    dp, pp, tp, r_ext, n_ext, mb = strat
    return ExecNode("_approx", ExecNodeType.OP, (Allocation((0, 0, 0), (r_ext, n_ext, g_ext)),),
                    op=UnrolledNode(v, 0), model=v.kind.model, pi=(dp, pp, tp), mb=mb)


@dataclass
class CandidateDirectory:
    """Per vertex: strategies sorted by isolated time, and the position of each strategy."""
    table: Dict[str, List[Tuple[int, int, int, int, int, int, float]]] = field(default_factory=dict)
    index: Dict[str, Dict[Strategy, int]] = field(default_factory=dict)

    def position(self, vid: str, plan: ExecutionPlan, stats: Optional[MoveStats] = None) -> int:
        dp, pp, tp = plan.pi[vid]
        r_ext, n_ext, _ = plan.sigma[vid].extent
        key = (dp, pp, tp, r_ext, n_ext, plan.mb[vid])
        pos = self.index[vid].get(key)
        if pos is None:
            if stats is not None:
                stats.n_fallback += 1
            return len(self.table[vid]) // 2
        return pos


def build_candidate_directory(rpeg: RPEG, suite: ModelSuite, space: DeviceSpace, workload: Workload,
                              cost_model: NodeCostModel, mem_model: NodeMemoryModel, max_per_vertex: int = 1000,
                              flags: Optional[SearchFlags] = None) -> CandidateDirectory:
    out = CandidateDirectory()
    cap = mem_model.capacity()
    for v in rpeg.vertices:
        rows = []
        for strat in enumerate_strategies(v, suite, space, workload, flags):
            g_ext = packing_geometry(strat[0], strat[1], strat[2], space.G)[0]
            node = mock_node(v, strat, g_ext)
            if mem_model.peak_bytes(node) > cap:
                continue
            rows.append(strat + (cost_model.time(node),))
        rows.sort(key=lambda c: c[6])
        rows = rows[:max_per_vertex]
        out.table[v.id] = rows
        out.index[v.id] = {c[:6]: j for j, c in enumerate(rows)}
    return out


def critical_chain(executable: ExecutableRPEG, trace: Trace) -> Set[ExecNode]:
    """Walk back from the last-finishing node through the latest-finishing predecessor."""
    pred: Dict[ExecNode, List[ExecNode]] = {n: [] for n in executable.nodes}
    for e in executable.edges:
        pred[e.dst].append(e.src)
    cur = max(executable.nodes, key=lambda n: trace.finish[n])
    chain = {cur}
    while pred[cur]:
        cur = max(pred[cur], key=lambda n: trace.finish[n])
        chain.add(cur)
    return chain


def critical_mass(chain: Set[ExecNode], rpeg: RPEG, trace: Trace) -> Dict[str, float]:
    mass = {v.id: 0.0 for v in rpeg.vertices}
    for n in chain:
        if n.kind is ExecNodeType.OP:
            mass[n.template_id] += trace.finish[n] - trace.start[n]
    return mass


def _with(config: Configuration, targets: Sequence[str], alloc: Allocation, pi, mb) -> Configuration:
    plan = config.plan.copy()
    for t in targets:
        plan.sigma[t], plan.pi[t], plan.mb[t] = alloc, pi, mb
    return Configuration(config.rpeg, plan, config.device_space, config.intra_stage_fusion, config.transfer_resource_policy)


def move_gen(config: Configuration, executable: ExecutableRPEG, trace: Trace, directory: CandidateDirectory, K_x: int,
             T_max: int, T: float, T_init: float, rng: random.Random, stats: Optional[MoveStats] = None,
             flags: Optional[SearchFlags] = None) -> List[Configuration]:
    """Up to ``K_x`` neighbours that change one vertex (both members of a fused training pair)."""
    verts = list(config.rpeg.vertices)
    uniform = flags is not None and flags.uniform_vertex
    if not uniform and rng.random() >= 0.4:
        mass = critical_mass(critical_chain(executable, trace), config.rpeg, trace)
        v = rng.choices(verts, weights=[mass[x.id] + 1e-6 for x in verts], k=1)[0]
    else:
        v = rng.choice(verts)
    rows = directory.table[v.id]
    space = config.device_space
    targets = [v.id]
    peer_rows = None
    if config.intra_stage_fusion and v.id in ("t_pi", "t_V"):
        peer = "t_V" if v.id == "t_pi" else "t_pi"
        if peer in config.plan.sigma:
            targets.append(peer)
            peer_rows = {(c[0], c[1], c[2], c[5]) for c in directory.table[peer]}
    out: List[Configuration] = []
    seen = set()
    cur_alloc, cur_pi, cur_mb = config.plan.sigma[v.id], config.plan.pi[v.id], config.plan.mb[v.id]
    for _ in range(min(5, T_max)):  # at most one pure re-placement
        o = sample_origin(rng, cur_alloc.extent, space)
        if o is not None and o != cur_alloc.origin:
            seen.add((cur_pi, o, cur_mb))
            out.append(_with(config, targets, Allocation(o, cur_alloc.extent), cur_pi, cur_mb))
            break
    if rows:
        w = max(5, int(len(rows) * min(1.0, T / T_init)))
        j_star = directory.position(v.id, config.plan, stats)
        lo, hi = max(0, j_star - w), min(len(rows) - 1, j_star + w)
        for _ in range(T_max):
            if len(out) >= K_x:
                break
            j = rng.randint(lo, hi)
            if j == j_star:
                continue
            dp, pp, tp, r_ext, n_ext, mb, _t = rows[j]
            geom = packing_geometry(dp, pp, tp, space.G)
            if geom is None or (peer_rows is not None and (dp, pp, tp, mb) not in peer_rows):
                continue
            extent = (r_ext, n_ext, geom[0])
            o = sample_origin(rng, extent, space)
            key = ((dp, pp, tp), o, mb)
            if o is None or key in seen:
                continue
            seen.add(key)
            out.append(_with(config, targets, Allocation(o, extent), (dp, pp, tp), mb))
    if stats is not None:
        stats.n_calls += 1
        for c in out:
            if c.plan.pi == config.plan.pi and c.plan.mb == config.plan.mb:
                stats.n_placement_proposed += 1
            else:
                stats.n_strategy_proposed += 1
        if not out:
            stats.n_empty += 1
    return out


def multi_move_pair(config: Configuration, suite: ModelSuite, workload: Workload, rng: random.Random,
                    max_retries: int = 100, flags: Optional[SearchFlags] = None) -> Optional[Configuration]:
    """Donor (chosen by device count) gives up racks; a vertex overlapping it is re-sampled over its
    own racks plus the freed ones. Fused training pairs do not take part."""
    verts = list(config.rpeg.vertices)
    space = config.device_space
    plan = config.plan
    sizes = [float(plan.sigma[v.id].size()) for v in verts]
    if sum(sizes) == 0:
        return None
    donor = rng.choices(verts, weights=sizes, k=1)[0]
    receivers = [v for v in verts if v.id != donor.id and plan.sigma[v.id].overlaps(plan.sigma[donor.id])]
    if not receivers:
        return None
    receiver = rng.choice(receivers)
    if config.intra_stage_fusion and {donor.id, receiver.id} & {"t_pi", "t_V"}:
        return None
    d_alloc = plan.sigma[donor.id]
    d_lo, d_hi = d_alloc.origin[0], d_alloc.origin[0] + d_alloc.extent[0]
    if d_hi - d_lo > 1:
        keep = rng.randint(1, d_hi - d_lo - 1)
        start = rng.randint(d_lo, d_hi - keep)
        new_lo, new_hi = start, start + keep
    else:
        new_lo, new_hi = d_lo, d_hi
    new_d = None
    for _ in range(max_retries):
        new_d = sample_strategy(rng, donor, suite, space, workload, new_lo, new_hi, flags)
        if new_d is not None:
            break
    if new_d is None:
        return None
    r_alloc = plan.sigma[receiver.id]
    freed = set(range(d_lo, d_hi)) - set(range(new_lo, new_hi))
    racks = set(range(r_alloc.origin[0], r_alloc.origin[0] + r_alloc.extent[0])) | freed
    lo, hi = min(racks), max(racks) + 1
    if set(range(lo, hi)) != racks:  # not contiguous: fall back to the whole machine
        lo, hi = 0, space.R
    new_r = None
    for _ in range(max_retries):
        new_r = sample_strategy(rng, receiver, suite, space, workload, lo, hi, flags)
        if new_r is not None:
            break
    if new_r is None:
        return None
    out = plan.copy()
    for vid, (alloc, pi, mb) in ((donor.id, new_d), (receiver.id, new_r)):
        out.sigma[vid], out.pi[vid], out.mb[vid] = alloc, pi, mb
    return Configuration(config.rpeg, out, space, config.intra_stage_fusion, config.transfer_resource_policy)
