"""Per-node GPU preflight inside a Slurm allocation, and the cluster contract that compares the nodes.

    srun --ntasks-per-node=1 python -m rpeg_b200.runtime.slurm_preflight --expected-gpus 8 >> preflight.jsonl
    python -m rpeg_b200.runtime.slurm_preflight --contract-from preflight.jsonl --contract-output contract.json

Step one runs once on every node and prints ONE JSON line: host name, the GPUs torch and ``nvidia-smi`` see (count,
names, memory), driver / torch / CUDA / NCCL versions, NIC firmware, the node's wall clock; exit code 2 when the node
does not have the expected number of healthy GPUs. Step two reads the lines of all nodes and writes
``rpeg.cluster_contract.v1``: whether the nodes are comparable for performance work (one driver, one CUDA, one NCCL,
one NIC firmware set, clocks within ``--max-clock-skew-s``), with the reasons when they are not.
``hardware_from_preflight`` turns the same lines into the ``(gpu type, smallest GPU memory)`` a job is planned with.

Everything here only READS: ``nvidia-smi --query-gpu`` for names, memory and driver; no GPU setting is changed.
The probes are plain functions passed in by the caller, so the logic is tested without GPUs.

Reference: RPEG/runtime/slurm_preflight.py:63-275 (node health :63-186, contract :187-234, hardware resolution :237-275).
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

from .errors import RuntimeConfigError

CONTRACT_SCHEMA = "rpeg.cluster_contract.v1"


@dataclass
class NodeReport:
    hostname: str
    expected_gpus: int
    ok: bool = False
    message: str = ""
    cuda_visible_devices: Optional[str] = None
    torch_cuda_available: bool = False
    torch_device_count: int = 0
    smi_device_count: Optional[int] = None
    device_names: List[str] = field(default_factory=list)
    total_memory_bytes: List[int] = field(default_factory=list)
    compute_capabilities: List[str] = field(default_factory=list)
    driver_version: Optional[str] = None
    torch_version: Optional[str] = None
    torch_cuda_version: Optional[str] = None
    nccl_version: Optional[str] = None
    nic_firmware: List[str] = field(default_factory=list)
    wall_time_ns: int = 0

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d["min_total_memory_bytes"] = min(self.total_memory_bytes) if self.total_memory_bytes else None
        return d


# ------------------------------------------------------------------------------------------------ probes
def probe_torch() -> Dict[str, Any]:
    """What torch sees on this node (never raises)."""
    out: Dict[str, Any] = {"available": False, "count": 0, "names": [], "memory": [], "capabilities": [],
                           "torch_version": None, "cuda_version": None, "nccl_version": None}
    try:
        import torch
        out["torch_version"] = str(torch.__version__)
        out["cuda_version"] = str(torch.version.cuda)
        try:
            out["nccl_version"] = ".".join(str(p) for p in torch.cuda.nccl.version())
        except Exception:
            pass
        if torch.cuda.is_available():
            out["available"] = True
            out["count"] = torch.cuda.device_count()
            for i in range(out["count"]):
                p = torch.cuda.get_device_properties(i)
                out["names"].append(p.name)
                out["memory"].append(int(p.total_memory))
                out["capabilities"].append(f"{p.major}.{p.minor}")
    except Exception as exc:          # a broken installation is a finding, not a crash
        out["error"] = str(exc)
    return out


def probe_smi() -> Dict[str, Any]:
    """``nvidia-smi --query-gpu=name,memory.total,driver_version`` (read only); ``{"count": None}`` without the tool."""
    exe = shutil.which("nvidia-smi")
    if exe is None:
        return {"count": None, "driver": None, "error": "nvidia-smi not found"}
    try:
        r = subprocess.run([exe, "--query-gpu=name,memory.total,driver_version", "--format=csv,noheader,nounits"],
                           capture_output=True, text=True, timeout=60)
    except Exception as exc:
        return {"count": None, "driver": None, "error": str(exc)}
    if r.returncode != 0:
        return {"count": None, "driver": None, "error": (r.stderr or r.stdout).strip()[:200]}
    rows = [[c.strip() for c in line.split(",")] for line in r.stdout.splitlines() if line.strip()]
    drivers = sorted({row[2] for row in rows if len(row) >= 3})
    return {"count": len(rows), "driver": drivers[0] if len(drivers) == 1 else (",".join(drivers) or None),
            "names": [row[0] for row in rows], "memory_mib": [int(float(row[1])) for row in rows if len(row) >= 2]}


def probe_nic_firmware(root: str = "/sys/class/infiniband") -> List[str]:
    """``device:firmware`` of every RDMA NIC the kernel lists (empty on a single-node NVSwitch box without them)."""
    out: List[str] = []
    base = Path(root)
    if base.is_dir():
        for dev in sorted(base.iterdir()):
            try:
                out.append(f"{dev.name}:{(dev / 'fw_ver').read_text().strip()}")
            except OSError:
                continue
    return out


# ------------------------------------------------------------------------------------------------ node health
def check_node(expected_gpus: int, *, torch_probe: Callable[[], Dict[str, Any]] = probe_torch,
               smi_probe: Callable[[], Dict[str, Any]] = probe_smi, nic_probe: Callable[[], List[str]] = probe_nic_firmware,
               hostname: Optional[str] = None, clock_ns: Callable[[], int] = time.time_ns,
               min_memory_bytes: int = 0, require_capability: Optional[str] = None) -> NodeReport:
    """The node passes when torch sees exactly ``expected_gpus`` devices, ``nvidia-smi`` (if present) agrees, every
    GPU has at least ``min_memory_bytes`` and, if asked, the compute capability ``require_capability`` (``"10.0"``)."""
    t, s = torch_probe(), smi_probe()
    rep = NodeReport(hostname=hostname or os.uname().nodename, expected_gpus=int(expected_gpus),
                     cuda_visible_devices=os.environ.get("CUDA_VISIBLE_DEVICES"),
                     torch_cuda_available=bool(t.get("available")), torch_device_count=int(t.get("count") or 0),
                     smi_device_count=s.get("count"), device_names=list(t.get("names") or []),
                     total_memory_bytes=[int(x) for x in (t.get("memory") or [])],
                     compute_capabilities=list(t.get("capabilities") or []), driver_version=s.get("driver"),
                     torch_version=t.get("torch_version"), torch_cuda_version=t.get("cuda_version"),
                     nccl_version=t.get("nccl_version"), nic_firmware=list(nic_probe()), wall_time_ns=int(clock_ns()))
    problems: List[str] = []
    if t.get("error"):
        problems.append(f"torch: {t['error']}")
    if not rep.torch_cuda_available:
        problems.append("torch sees no CUDA device")
    if rep.torch_device_count != rep.expected_gpus:
        problems.append(f"torch sees {rep.torch_device_count} GPU(s), expected {rep.expected_gpus}")
    visible_all = rep.cuda_visible_devices in (None, "")
    if rep.smi_device_count is not None and visible_all and rep.smi_device_count != rep.torch_device_count:
        problems.append(f"nvidia-smi lists {rep.smi_device_count} GPU(s), torch {rep.torch_device_count}")
    small = [i for i, m in enumerate(rep.total_memory_bytes) if m < min_memory_bytes]
    if small:
        problems.append(f"GPU(s) {small} have less than {min_memory_bytes} bytes")
    if require_capability is not None:
        wrong = [i for i, c in enumerate(rep.compute_capabilities) if c != require_capability]
        if wrong:
            problems.append(f"GPU(s) {wrong} are not compute capability {require_capability}")
    if len(set(rep.device_names)) > 1:
        problems.append(f"mixed GPU models on one node: {sorted(set(rep.device_names))}")
    rep.ok = not problems
    rep.message = "ok" if rep.ok else "; ".join(problems)
    return rep


# ------------------------------------------------------------------------------------------------ contract
def read_rows(path) -> List[Dict[str, Any]]:
    rows = []
    for n, line in enumerate(Path(path).read_text().splitlines(), 1):
        if not line.strip():
            continue
        try:
            rows.append(json.loads(line))
        except json.JSONDecodeError as exc:
            raise RuntimeConfigError(f"{path}:{n}: not a JSON line ({exc})") from None
    return rows


def cluster_contract(rows: Sequence[Dict[str, Any]], *, max_clock_skew_s: float = 1.0, expected_nodes: Optional[int] = None) -> Dict[str, Any]:
    """Are the nodes comparable? One value per software layer across the nodes, clocks within the bound, every node
    healthy, no node reported twice, and (if given) the expected number of nodes."""
    def distinct(key: str) -> List[str]:
        return sorted({str(r[key]) for r in rows if r.get(key)})

    drivers, cudas, nccls, torches = distinct("driver_version"), distinct("torch_cuda_version"), distinct("nccl_version"), distinct("torch_version")
    firmware = sorted({tuple(str(x) for x in (r.get("nic_firmware") or ())) for r in rows})
    gpu_models = sorted({str(n) for r in rows for n in (r.get("device_names") or ())})
    clocks = [int(r["wall_time_ns"]) for r in rows if r.get("wall_time_ns")]
    skew = (max(clocks) - min(clocks)) / 1e9 if len(clocks) >= 2 else 0.0
    hosts = [str(r.get("hostname") or "") for r in rows]
    reasons: List[str] = []
    for what, values in (("NVIDIA driver versions", drivers), ("CUDA versions", cudas), ("NCCL versions", nccls),
                         ("torch versions", torches), ("GPU models", gpu_models)):
        if len(values) > 1:
            reasons.append(f"heterogeneous {what}: {values}")
    if len(firmware) > 1:
        reasons.append("heterogeneous NIC firmware")
    if skew > float(max_clock_skew_s):
        reasons.append(f"node clock skew {skew:.6f} s exceeds {float(max_clock_skew_s):.6f} s")
    unhealthy = sorted(h for h, r in zip(hosts, rows) if not r.get("ok"))
    if unhealthy:
        reasons.append(f"unhealthy nodes: {unhealthy}")
    dup = sorted({h for h in hosts if hosts.count(h) > 1})
    if dup:
        reasons.append(f"nodes reported more than once: {dup}")
    if expected_nodes is not None and len(rows) != int(expected_nodes):
        reasons.append(f"{len(rows)} node report(s), expected {int(expected_nodes)}")
    mems = [int(r["min_total_memory_bytes"]) for r in rows if r.get("min_total_memory_bytes")]
    return {"schema_version": CONTRACT_SCHEMA, "nodes": len(rows), "hostnames": sorted(hosts), "driver_versions": drivers,
            "torch_cuda_versions": cudas, "nccl_versions": nccls, "torch_versions": torches, "gpu_models": gpu_models,
            "nic_firmware_sets": [list(f) for f in firmware], "gpus_per_node": sorted({int(r.get("torch_device_count") or 0) for r in rows}),
            "min_gpu_memory_bytes": min(mems) if mems else None, "clock_skew_s": skew, "max_clock_skew_s": float(max_clock_skew_s),
            "performance_comparable": not reasons, "non_comparable_reasons": reasons}


def hardware_from_preflight(rows: Optional[Sequence[Dict[str, Any]]], *, expected_nodes: int, explicit_memory_bytes: Optional[int] = None,
                            explicit_gpu_type: Optional[str] = None) -> Tuple[str, int]:
    """``(gpu type, bytes of the smallest GPU)`` to plan a job with: from the preflight lines when there are any
    (every expected node must have reported its memory), else from the explicit values of the job file."""
    if rows:
        caps = [int(r["min_total_memory_bytes"]) for r in rows if r.get("min_total_memory_bytes")]
        if len(caps) != int(expected_nodes):
            raise RuntimeConfigError(f"GPU preflight reported memory for {len(caps)} of {expected_nodes} node(s)")
        names = sorted({str(n) for r in rows for n in (r.get("device_names") or ()) if n})
        return ",".join(names) or "unknown", min(caps)
    if explicit_memory_bytes is None:
        raise RuntimeConfigError("GPU memory is unknown: run the preflight or give hardware.memory_per_gpu explicitly")
    if int(explicit_memory_bytes) <= 0:
        raise RuntimeConfigError("explicit GPU memory must be positive")
    return explicit_gpu_type or "explicit", int(explicit_memory_bytes)


# ------------------------------------------------------------------------------------------------ CLI
def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="GPU health of this node (one JSON line), or the contract over all nodes' lines")
    ap.add_argument("--expected-gpus", type=int)
    ap.add_argument("--min-memory-bytes", type=int, default=0)
    ap.add_argument("--require-capability", default=None, help='e.g. "10.0" for B200')
    ap.add_argument("--contract-from", help="file with the JSON lines of all nodes")
    ap.add_argument("--contract-output")
    ap.add_argument("--expected-nodes", type=int)
    ap.add_argument("--max-clock-skew-s", type=float, default=1.0)
    ap.add_argument("--strict", action="store_true", help="with --contract-from: exit 2 when the nodes are not comparable")
    args = ap.parse_args(argv)
    if args.contract_from:
        try:
            contract = cluster_contract(read_rows(args.contract_from), max_clock_skew_s=args.max_clock_skew_s, expected_nodes=args.expected_nodes)
        except (OSError, RuntimeConfigError) as exc:
            print(f"preflight error: {exc}", file=sys.stderr)
            return 2
        text = json.dumps(contract, indent=2, sort_keys=True) + "\n"
        if args.contract_output:
            Path(args.contract_output).write_text(text)
        print(text, end="", flush=True)
        return 2 if (args.strict and not contract["performance_comparable"]) else 0
    if args.expected_gpus is None:
        ap.error("--expected-gpus is required unless --contract-from is given")
    rep = check_node(args.expected_gpus, min_memory_bytes=args.min_memory_bytes, require_capability=args.require_capability)
    print(json.dumps(rep.to_dict(), sort_keys=True), flush=True)
    return 0 if rep.ok else 2


if __name__ == "__main__":
    sys.exit(main())
