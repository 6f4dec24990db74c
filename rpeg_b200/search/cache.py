"""Evaluation cache keyed by a canonical hash of (RPEG structure, plan).

``config_hash`` is the sha256 of a canonical JSON description: vertex ids with role/model,
staleness, and per-vertex placement, parallelism and microbatch count; ``EvalCache`` stores
``(score, trace, feasible)`` and counts hits and misses (reference: RPEG/search/cache.py:22-185).
"""
from __future__ import annotations

import hashlib
import json
from typing import Dict, Optional, Tuple

from ..ir.plan import ExecutionPlan
from ..ir.rpeg import RPEG


def config_hash(rpeg: RPEG, plan: ExecutionPlan) -> str:
    body = {
        "vertices": [[v.id, v.kind.role.value, v.kind.model.value] for v in rpeg.vertices],
        "tau": sorted((m.value, int(t)) for m, t in rpeg.tau.items()),
        "plan": [[v.id, list(plan.sigma[v.id].origin), list(plan.sigma[v.id].extent), list(plan.pi[v.id]),
                  int(plan.mb.get(v.id, 1))] for v in rpeg.vertices if v.id in plan.sigma],
    }
    return hashlib.sha256(json.dumps(body, sort_keys=True, separators=(",", ":")).encode()).hexdigest()


class EvalCache:
    def __init__(self, max_entries: Optional[int] = None):
        self._data: Dict[str, Tuple[float, object, bool]] = {}
        self.hits = 0
        self.misses = 0
        self.max_entries = max_entries

    def __contains__(self, key: str) -> bool:
        return key in self._data

    def __len__(self) -> int:
        return len(self._data)

    def get(self, key: str):
        self.hits += 1
        return self._data[key]

    def put(self, key: str, score: float, trace, feasible: bool) -> None:
        self.misses += 1
        if self.max_entries is not None and len(self._data) >= self.max_entries:
            self._data.pop(next(iter(self._data)))
        self._data[key] = (score, trace, feasible)

    def hit_rate(self) -> float:
        total = self.hits + self.misses
        return self.hits / total if total else 0.0

    def stats(self) -> dict:
        return {"hits": self.hits, "misses": self.misses, "hit_rate": self.hit_rate(), "entries": len(self._data)}
