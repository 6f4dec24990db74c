"""Mapping of logical grid coordinates (rack, node, gpu) to physical devices.

On one NVSwitch node the inventory is simply ``cuda:0..G-1`` on localhost; the file form exists so
that a plan made for a logical grid can be executed on any host list (reference:
RPEG/runtime/cluster.py:24-158)."""
from __future__ import annotations

import os
import socket
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

from ..core.types import Allocation, DeviceSpace
from .errors import RuntimeConfigError
from .io import load_mapping


@dataclass(frozen=True)
class GPURef:
    hostname: str
    local_cuda_index: int
    global_rank: int
    coord: Tuple[int, int, int]


class ClusterInventory:
    def __init__(self, space: DeviceSpace, gpus: Dict[Tuple[int, int, int], GPURef]):
        self.space, self.gpus = space, gpus
        missing = [(r, n, g) for r in range(space.R) for n in range(space.N) for g in range(space.G) if (r, n, g) not in gpus]
        if missing:
            raise RuntimeConfigError(f"inventory lacks devices for logical coordinates {missing[:8]}")

    def resolve_allocation(self, alloc: Allocation) -> Tuple[GPURef, ...]:
        if not alloc.fits(self.space):
            raise RuntimeConfigError(f"allocation {alloc} lies outside the device space")
        return tuple(self.gpus[c] for c in alloc.coords())

    def rank_of(self, coord: Tuple[int, int, int]) -> int:
        return self.gpus[coord].global_rank


def local_inventory(space: DeviceSpace, hostname: Optional[str] = None) -> ClusterInventory:
    """Every logical device on this host; logical GPU (r, n, g) is rank ``device_id`` and CUDA index
    ``device_id`` modulo the visible device count (a grid larger than the machine is still usable for
    dry runs and metadata execution)."""
    host = hostname or socket.gethostname()
    visible = max(1, int(os.environ.get("RPEG_VISIBLE_GPUS", "0")) or space.num_devices())
    gpus = {}
    for r in range(space.R):
        for n in range(space.N):
            for g in range(space.G):
                rank = space.device_id(r, n, g)
                gpus[(r, n, g)] = GPURef(host, rank % visible, rank, (r, n, g))
    return ClusterInventory(space, gpus)


def inventory_from_file(path, space: DeviceSpace) -> ClusterInventory:
    raw = load_mapping(path)
    gpus = {}
    for entry in raw.get("devices", []):
        coord = tuple(int(x) for x in entry["coord"])
        gpus[coord] = GPURef(str(entry["hostname"]), int(entry["cuda_index"]), int(entry.get("rank", space.device_id(*coord))), coord)
    return ClusterInventory(space, gpus)
