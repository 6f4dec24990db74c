"""Result of scheduling an executable graph: start/finish time per node plus the device
allocations each node kept busy. Scores follow the reference (RPEG/schedule/trace.py:31-118):
``makespan`` is the latest finish, ``throughput = K * W_step / makespan`` and ``utilization`` is
the mean over used devices of (merged busy time / makespan)."""
from __future__ import annotations

from collections import defaultdict
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

from ..core.types import Allocation
from ..passes.lower import ExecNode, ExecNodeType


@dataclass(frozen=True)
class Trace:
    start: Dict[ExecNode, float]
    finish: Dict[ExecNode, float]
    reserved_allocations: Optional[Dict[ExecNode, Tuple[Allocation, ...]]] = None
    dispatch_order: Optional[Tuple[ExecNode, ...]] = None   # nodes in the order the scheduler placed them

    def makespan(self) -> float:
        return max(self.finish.values())

    def throughput(self, W_step: float, K: int) -> float:
        return K * W_step / self.makespan()

    def seconds_by_kind(self) -> Dict[str, float]:
        """Scheduled duration summed per operator role (``GEN``, ``INF``, ``TRAIN``) and per transfer kind
        (``comm``, ``reshard``): what a measured trace's per-class totals are compared with."""
        out: Dict[str, float] = defaultdict(float)
        for node, s in self.start.items():
            key = node.role.value if node.kind is ExecNodeType.OP and node.role is not None else node.kind.value
            out[key] += self.finish[node] - s
        return dict(out)

    def seconds_by_vertex(self) -> Dict[str, float]:
        """Scheduled duration of the operator nodes summed per template vertex (``g_pi``, ``i_ref``, ``t_pi``, ...)
        over all logical steps and quantile phases."""
        out: Dict[str, float] = defaultdict(float)
        for node, s in self.start.items():
            if node.kind is ExecNodeType.OP:
                out[node.template_id or node.id] += self.finish[node] - s
        return dict(out)

    def _busy_allocs(self, node: ExecNode) -> Tuple[Allocation, ...]:
        if self.reserved_allocations is not None:
            return self.reserved_allocations[node]
        if node.kind in (ExecNodeType.COMM, ExecNodeType.RESHARD):
            return node.allocs[-1:]
        return node.allocs

    def utilization(self) -> float:
        span = self.makespan()
        if span <= 0:
            return 0.0
        spans = defaultdict(list)
        for node, s in self.start.items():
            for alloc in self._busy_allocs(node):
                for dev in alloc.coords():
                    spans[dev].append((s, self.finish[node]))
        if not spans:
            return 0.0
        total = 0.0
        for intervals in spans.values():
            busy, cur_s, cur_e = 0.0, None, None
            for s, e in sorted(intervals):
                if cur_e is None or s > cur_e:
                    if cur_e is not None:
                        busy += cur_e - cur_s
                    cur_s, cur_e = s, e
                else:
                    cur_e = max(cur_e, e)
            if cur_e is not None:
                busy += cur_e - cur_s
            total += busy / span
        return total / len(spans)

    def n_active(self) -> int:
        devs = set()
        for node in self.start:
            for alloc in node.allocs:
                devs.update(alloc.coords())
        return len(devs)

    def ordered(self):
        """Nodes by (start, finish, id): the dispatch order a runtime should follow."""
        if self.dispatch_order is not None:
            return list(self.dispatch_order)
        return sorted(self.start, key=lambda n: (self.start[n], self.finish[n], n.id))
