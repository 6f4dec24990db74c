"""Execution plan: placement ``sigma``, parallelism ``pi = (dp, pp, tp)`` and microbatch count
``mb`` per template vertex (reference: RPEG/ir/plan.py:16)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Tuple

from ..core.types import Allocation


@dataclass
class ExecutionPlan:
    sigma: Dict[str, Allocation] = field(default_factory=dict)
    pi: Dict[str, Tuple[int, int, int]] = field(default_factory=dict)
    mb: Dict[str, int] = field(default_factory=dict)

    def copy(self) -> "ExecutionPlan":
        return ExecutionPlan(dict(self.sigma), dict(self.pi), dict(self.mb))

    def fingerprint(self) -> tuple:
        return tuple(sorted((v, self.pi[v], self.sigma[v].origin, self.sigma[v].extent, self.mb.get(v, 1))
                            for v in self.sigma))
