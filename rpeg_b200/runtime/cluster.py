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


def expand_nodelist(nodelist: str) -> Tuple[str, ...]:
    """Host names of a Slurm node list such as ``gpu[01-03,07],login1`` (what ``scontrol show hostnames`` prints)."""
    hosts, depth, cur = [], 0, ""
    for ch in nodelist.strip() + ",":
        if ch == "[":
            depth += 1
        elif ch == "]":
            depth -= 1
        if ch == "," and depth == 0:
            if cur:
                hosts.append(cur)
            cur = ""
        else:
            cur += ch
    out = []
    for h in hosts:
        if "[" not in h:
            out.append(h)
            continue
        prefix, rest = h.split("[", 1)
        body, suffix = rest.rsplit("]", 1)
        for part in body.split(","):
            if "-" in part:
                lo, hi = part.split("-", 1)
                width = len(lo)
                out.extend(f"{prefix}{i:0{width}d}{suffix}" for i in range(int(lo), int(hi) + 1))
            else:
                out.append(f"{prefix}{part}{suffix}")
    return tuple(out)


def slurm_inventory(space: DeviceSpace, env: Optional[Dict[str, str]] = None) -> ClusterInventory:
    """Inventory of a Slurm allocation from its environment: node ``i`` of ``SLURM_JOB_NODELIST`` is logical node
    ``i`` (racks filled first to last), its GPUs are CUDA indices ``0..G-1``; ranks follow the logical device id,
    which is the order ``torch.distributed.run --node-rank $SLURM_NODEID`` gives them (reference:
    RPEG/runtime/cluster.py:89-111)."""
    env = os.environ if env is None else env
    nodelist = env.get("SLURM_JOB_NODELIST") or env.get("SLURM_NODELIST")
    if not nodelist:
        raise RuntimeConfigError("no SLURM_JOB_NODELIST in the environment")
    hosts = expand_nodelist(nodelist)
    need = space.R * space.N
    if len(hosts) < need:
        raise RuntimeConfigError(f"the plan needs {need} node(s), the Slurm allocation has {len(hosts)}")
    gpus = {}
    for r in range(space.R):
        for n in range(space.N):
            host = hosts[r * space.N + n]
            for g in range(space.G):
                gpus[(r, n, g)] = GPURef(host, g, space.device_id(r, n, g), (r, n, g))
    return ClusterInventory(space, gpus)
