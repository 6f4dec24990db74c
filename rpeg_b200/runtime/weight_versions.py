"""Weight-version arithmetic of bounded staleness.

Logical steps are 1-based. Version 0 is the initial weights; training in step ``s`` produces version
``s``. A consumer of model ``m`` with staleness ``tau`` running in step ``s`` reads version
``max(0, s - 1 - tau)``, the runtime counterpart of the unroll rule ``s_m(k) = max(0, k - (tau+1))``
on 0-based iterations (reference: RPEG/runtime/weight_versions.py:25-30, RPEG/runtime/dataflow.md:74-81)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional


def consumer_weight_version(step: int, tau: int) -> int:
    if step < 1 or tau < 0:
        raise ValueError("step is 1-based and tau is non-negative")
    return max(0, step - 1 - tau)


def producer_weight_version(step: int) -> int:
    return step


def uses_shadow_copies(tau: int) -> bool:
    """A positive staleness budget means the serving side keeps its own (older) copy on other devices."""
    return tau > 0


@dataclass
class WeightVersionTable:
    """Which versions of each model are currently materialised, and who still needs them."""
    keep_latest: int = 8
    versions: Dict[str, List[int]] = field(default_factory=dict)
    pins: Dict[str, Dict[int, int]] = field(default_factory=dict)

    def publish(self, model: str, version: int) -> None:
        vs = self.versions.setdefault(model, [])
        if version not in vs:
            vs.append(version)
            vs.sort()

    def latest(self, model: str) -> Optional[int]:
        vs = self.versions.get(model)
        return vs[-1] if vs else None

    def has(self, model: str, version: int) -> bool:
        return version in self.versions.get(model, [])

    def pin(self, model: str, version: int) -> None:
        d = self.pins.setdefault(model, {})
        d[version] = d.get(version, 0) + 1

    def unpin(self, model: str, version: int) -> None:
        d = self.pins.get(model, {})
        if d.get(version, 0) <= 1:
            d.pop(version, None)
        else:
            d[version] -= 1

    def prune(self, model: str, needed: Optional[set] = None) -> List[int]:
        """Drop versions beyond ``keep_latest`` that nobody pins or still needs; returns what was dropped."""
        vs = self.versions.get(model, [])
        keep = set(vs[-self.keep_latest:]) | set(self.pins.get(model, {})) | set(needed or ())
        dropped = [v for v in vs if v not in keep]
        self.versions[model] = [v for v in vs if v in keep]
        return dropped
