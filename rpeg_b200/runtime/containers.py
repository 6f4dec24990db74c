"""Runtime handles for data containers: which rows of which logical array live where.

Rows of rollout artefacts (completion ids, log-probs, values, rewards) are identified by their
global sample index so that partial, out-of-order arrival from quantile phases is well defined
(reference: RPEG/runtime/containers.py, RPEG/runtime/dataflow.md:12-26)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


@dataclass(frozen=True)
class ShardingSpec:
    dp: int = 1
    pp: int = 1
    tp: int = 1

    def rows_of(self, dp_rank: int, n_rows: int) -> range:
        per = n_rows // self.dp
        return range(dp_rank * per, (dp_rank + 1) * per)


@dataclass(frozen=True)
class ContainerRef:
    name: str
    step: int
    part: Optional[int] = None          # quantile phase index, None = whole container
    n_rows: int = 0
    nbytes: int = 0
    producer: Optional[str] = None
    weight_version: Optional[int] = None

    @property
    def key(self) -> Tuple[str, int, Optional[int]]:
        return (self.name, self.step, self.part)


@dataclass(frozen=True)
class WeightVersion:
    model: str
    version: int
    layout: Tuple[int, int, int]
    allocation: Optional[tuple] = None


class ContainerStore:
    """Metadata registry of produced containers; tensors themselves stay with the engine."""

    def __init__(self):
        self._refs: Dict[Tuple[str, int, Optional[int]], ContainerRef] = {}
        self.released: List[Tuple[str, int, Optional[int]]] = []

    def put(self, ref: ContainerRef) -> None:
        self._refs[ref.key] = ref

    def get(self, name: str, step: int, part: Optional[int] = None) -> ContainerRef:
        return self._refs[(name, step, part)]

    def parts(self, name: str, step: int) -> List[ContainerRef]:
        return sorted((r for r in self._refs.values() if r.name == name and r.step == step), key=lambda r: (r.part is None, r.part))

    def release_step(self, step: int) -> int:
        keys = [k for k in self._refs if k[1] == step]
        for k in keys:
            self.released.append(k)
            del self._refs[k]
        return len(keys)

    def __len__(self) -> int:
        return len(self._refs)
