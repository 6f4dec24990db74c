"""Core value types of the planner: device grid, allocations, containers, template graph pieces.

Same public surface as the reference's ``RPEG/core/types.py`` (enums at :88-127, the transfer
reservation policy at :128-200, ``DeviceSpace``/``Allocation``/``Container``/``OperatorKind``/
``TemplateVertex``/``TemplateEdge`` at :206-341 and ``packing_geometry`` at :16-85) so plans and
YAML written for either tool load in the other.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from enum import Enum
from typing import Iterator, Optional, Tuple


class Role(Enum):
    GENERATION = "GEN"
    INFERENCE = "INF"
    TRAINING = "TRAIN"


class Model(Enum):
    ACTOR = "Pi"
    CRITIC = "V"
    REFERENCE = "Ref"
    REWARD = "R"
    AC_SHARE = "AC"


class Collective(Enum):
    ALLREDUCE = "AllReduce"
    ALLGATHER = "AllGather"
    REDUCESCATTER = "ReduceScatter"
    ALLTOALL = "AllToAll"
    P2P = "PointToPoint"


class EdgeKind(Enum):
    DATA = "data"
    PUB = "pub"


_POLICY_VALUES = ("destination_only", "both_endpoints")


@dataclass(frozen=True)
class TransferResourcePolicy:
    """Which endpoints a COMM/RESHARD node keeps busy, separately for weights and activations."""

    weight: str = "destination_only"
    activation: str = "destination_only"

    def __post_init__(self) -> None:
        for field in (self.weight, self.activation):
            if field not in _POLICY_VALUES:
                raise ValueError(f"transfer resource policy must be one of {_POLICY_VALUES}, got {field!r}")

    def for_weight(self, is_weight: bool) -> str:
        return self.weight if is_weight else self.activation

    def to_dict(self) -> dict:
        return {"weight": self.weight, "activation": self.activation}

    @classmethod
    def from_dict(cls, data: Optional[dict]) -> "TransferResourcePolicy":
        if not data:
            return RPEG_TRANSFER_RESOURCE_POLICY
        return cls(weight=data.get("weight", "destination_only"), activation=data.get("activation", "destination_only"))


RPEG_TRANSFER_RESOURCE_POLICY = TransferResourcePolicy("destination_only", "destination_only")
CONSERVATIVE_TRANSFER_RESOURCE_POLICY = TransferResourcePolicy("both_endpoints", "both_endpoints")


def default_transfer_resource_policy() -> TransferResourcePolicy:
    name = os.environ.get("RPEG_TRANSFER_RESOURCE_POLICY", "").strip().lower()
    return CONSERVATIVE_TRANSFER_RESOURCE_POLICY if name == "conservative" else RPEG_TRANSFER_RESOURCE_POLICY


@dataclass(frozen=True)
class DeviceSpace:
    """Logical ``R`` racks x ``N`` nodes per rack x ``G`` GPUs per node."""

    R: int
    N: int
    G: int

    def num_devices(self) -> int:
        return self.R * self.N * self.G

    def device_id(self, r: int, n: int, g: int) -> int:
        return (r * self.N + n) * self.G + g


@dataclass(frozen=True)
class Allocation:
    """Axis-aligned box of devices: ``origin`` and ``extent`` are (racks, nodes, gpus)."""

    origin: Tuple[int, int, int]
    extent: Tuple[int, int, int]

    def size(self) -> int:
        r, n, g = self.extent
        return r * n * g

    def coords(self) -> Iterator[Tuple[int, int, int]]:
        (r0, n0, g0), (re, ne, ge) = self.origin, self.extent
        for r in range(r0, r0 + re):
            for n in range(n0, n0 + ne):
                for g in range(g0, g0 + ge):
                    yield (r, n, g)

    def device_ids(self, space: DeviceSpace) -> frozenset:
        return frozenset(space.device_id(*c) for c in self.coords())

    def fits(self, space: DeviceSpace) -> bool:
        return all(o >= 0 and e >= 1 and o + e <= lim
                   for o, e, lim in zip(self.origin, self.extent, (space.R, space.N, space.G)))

    def overlaps(self, other: "Allocation") -> bool:
        return all(a < b + be and b < a + ae
                   for a, ae, b, be in zip(self.origin, self.extent, other.origin, other.extent))

    def overlap_size(self, other: "Allocation") -> int:
        n = 1
        for a, ae, b, be in zip(self.origin, self.extent, other.origin, other.extent):
            n *= max(0, min(a + ae, b + be) - max(a, b))
        return n


@dataclass(frozen=True)
class Container:
    """Named data container: ``count`` elements of ``elem_size_bytes`` each."""

    name: str
    count: int
    elem_size_bytes: int

    def bytes(self) -> int:
        return self.count * self.elem_size_bytes


@dataclass(frozen=True)
class OperatorKind:
    role: Role
    model: Model
    read: Tuple[Container, ...] = ()
    write: Tuple[Container, ...] = ()


@dataclass(frozen=True)
class TemplateVertex:
    id: str
    kind: OperatorKind


@dataclass(frozen=True)
class TemplateEdge:
    src: TemplateVertex
    dst: TemplateVertex
    container: Container
    kind: EdgeKind = EdgeKind.DATA


def packing_geometry(dp: int, pp: int, tp: int, G: int) -> Optional[Tuple[int, int]]:
    """Shape ``(gpu_extent, node_count)`` of the box a (dp, pp, tp) strategy occupies, or ``None``.

    A TP group never leaves a node. ``s = min(pp, G // tp)`` pipeline stages share a node; the
    pipeline spans ``pp // s`` nodes (``pp`` must be divisible by ``s``). When a replica fits in one
    node, replicas either pack inside one node (``dp <= G // (s*tp)``) or fill whole nodes
    (``dp`` a multiple of the replicas per node). Reference: RPEG/core/types.py:16-57.
    """
    if min(dp, pp, tp, G) < 1 or tp > G:
        return None
    s = min(pp, G // tp)
    if s == 0 or pp % s:
        return None
    gpus_per_rep = s * tp
    nodes_per_rep = pp // s
    if nodes_per_rep == 1:
        reps_per_node = G // gpus_per_rep
        if reps_per_node == 0:
            return None
        if dp <= reps_per_node:
            return (dp * gpus_per_rep, 1)
        if dp % reps_per_node == 0:
            return (G, dp // reps_per_node)
        return None
    return (G, dp * nodes_per_rep)


def rectangular_node_layouts(nodes: int, R: int, N: int) -> list:
    """All ``(rack_extent, node_extent)`` with ``rack_extent * node_extent == nodes`` that fit R x N."""
    out = []
    for r_ext in range(1, min(R, nodes) + 1):
        if nodes % r_ext == 0 and nodes // r_ext <= N:
            out.append((r_ext, nodes // r_ext))
    return out
