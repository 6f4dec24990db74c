"""Launching the rank processes of a job on one node and tearing them down.

One process per GPU. ``LocalWorkerGroupLauncher`` starts ``world`` Python processes in a session of
their own (so the whole group can be signalled by process-group id and nothing else is touched),
gives each its rendezvous environment (loopback address, one port per job) and the JSON rank
assignment, waits for ``ready`` heartbeats and stops the group with SIGTERM followed by SIGKILL
after a grace period. ``torchrun_command`` renders the equivalent ``torch.distributed.run`` line for
a user who launches by hand. Reference: RPEG/runtime/launcher.py:27-211 (local launcher); the
reference's Slurm launcher (:212-407) is replaced by a batch file that `runtime.job_plan --emit-sbatch` writes
(one task per node running torchrun); the engine backend itself executes plans of one NVSwitch node.
"""
from __future__ import annotations

import json
import os
import signal
import subprocess
import sys
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Sequence

from .control import ControlPlane, HeartbeatStore
from .errors import RuntimeExecutionError


@dataclass(frozen=True)
class RankAssignment:
    rank: int
    local_rank: int
    hostname: str
    cuda_index: Optional[int]
    worker_ids: Sequence[str] = ()      # workers (model instances) this rank takes part in


@dataclass
class WorkerLaunch:
    group_id: str
    module: str                          # python module run with -m
    args: Sequence[str] = ()
    assignments: Sequence[RankAssignment] = ()
    master_port: int = 29531
    env: Dict[str, str] = field(default_factory=dict)
    log_dir: Optional[str] = None

    @property
    def world(self) -> int:
        return len(self.assignments)


def rank_environment(launch: WorkerLaunch, a: RankAssignment, heartbeat_dir: str) -> Dict[str, str]:
    env = dict(os.environ)
    env.update(launch.env)
    env.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(launch.master_port), "WORLD_SIZE": str(launch.world),
                "RANK": str(a.rank), "LOCAL_RANK": str(a.local_rank), "RPEG_GROUP_ID": launch.group_id,
                "RPEG_HEARTBEAT_DIR": str(heartbeat_dir),
                "RPEG_RANK_ASSIGNMENTS_JSON": json.dumps([asdict(x) for x in launch.assignments])})
    root = str(Path(__file__).resolve().parents[2])
    env["PYTHONPATH"] = root + (os.pathsep + env["PYTHONPATH"] if env.get("PYTHONPATH") else "")
    return env


def torchrun_command(module: str, args: Sequence[str], world: int, master_port: int = 29531) -> List[str]:
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
            "--master-port", str(master_port), "-m", module, *args]


class LocalWorkerGroupLauncher:
    def __init__(self, heartbeat_dir, poll_s: float = 0.02):
        self.heartbeat_dir = str(heartbeat_dir)
        self.store = HeartbeatStore(heartbeat_dir)
        self.control = ControlPlane(self.store, poll_s)
        self.procs: Dict[str, List[subprocess.Popen]] = {}
        self.launches: Dict[str, WorkerLaunch] = {}

    def launch(self, launch: WorkerLaunch) -> None:
        if launch.group_id in self.procs:
            raise RuntimeExecutionError(f"worker group {launch.group_id} is already running")
        procs = []
        for a in launch.assignments:
            out = subprocess.DEVNULL
            if launch.log_dir:
                Path(launch.log_dir).mkdir(parents=True, exist_ok=True)
                out = open(Path(launch.log_dir) / f"{launch.group_id}.rank{a.rank}.log", "w")
            procs.append(subprocess.Popen([sys.executable, "-m", launch.module, *launch.args], env=rank_environment(launch, a, self.heartbeat_dir),
                                          stdout=out, stderr=subprocess.STDOUT, start_new_session=True))
        self.procs[launch.group_id] = procs
        self.launches[launch.group_id] = launch

    def alive(self, group_id: str):
        procs = self.procs[group_id]
        return lambda rank: procs[rank].poll() is None

    def wait_ready(self, group_id: str, timeout_s: float = 120.0):
        try:
            return self.control.wait_for_state(group_id, self.launches[group_id].world, ("ready", "running", "finished"), timeout_s,
                                               alive=self.alive(group_id))
        except RuntimeExecutionError:
            self.stop(group_id, grace_s=1.0)      # a group that failed to come up is torn down as a whole
            raise

    def assert_healthy(self, group_id: str, stale_after_s: Optional[float] = None) -> None:
        self.control.assert_healthy(group_id, self.launches[group_id].world, alive=self.alive(group_id), stale_after_s=stale_after_s)

    def wait_finished(self, group_id: str, timeout_s: float) -> List[int]:
        deadline = time.monotonic() + timeout_s
        procs = self.procs[group_id]
        while any(p.poll() is None for p in procs):
            if any(p.poll() not in (None, 0) for p in procs):
                break
            if time.monotonic() > deadline:
                self.stop(group_id, grace_s=1.0)
                raise RuntimeExecutionError(f"{group_id}: ranks still running after {timeout_s:.1f}s")
            time.sleep(0.02)
        codes = [p.poll() for p in procs]
        if any(c not in (None, 0) for c in codes):
            self.stop(group_id, grace_s=1.0)       # one rank failed: abort the whole group
            bad = {r: c for r, c in enumerate(codes) if c not in (None, 0)}
            hb = {r: self.store.read(group_id, r) for r in bad}
            detail = {r: (None if hb[r] is None else hb[r].message) for r in bad}
            raise RuntimeExecutionError(f"{group_id}: rank(s) failed with exit codes {bad}: {detail}")
        return [int(c) for c in codes]

    def stop(self, group_id: str, grace_s: float = 5.0) -> None:
        """SIGTERM every rank's own process group, then SIGKILL what is left after the grace period."""
        procs = self.procs.pop(group_id, [])
        self.launches.pop(group_id, None)
        for sig, wait in ((signal.SIGTERM, grace_s), (signal.SIGKILL, 1.0)):
            live = [p for p in procs if p.poll() is None]
            if not live:
                break
            for p in live:
                try:
                    os.killpg(p.pid, sig)          # the rank is the leader of the session it was started in
                except (ProcessLookupError, PermissionError):
                    pass
            deadline = time.monotonic() + wait
            while time.monotonic() < deadline and any(p.poll() is None for p in live):
                time.sleep(0.02)
        for p in procs:
            if p.stdout not in (None, subprocess.DEVNULL) and hasattr(p.stdout, "close"):
                p.stdout.close()

    def stop_all(self) -> None:
        for g in list(self.procs):
            self.stop(g)


def single_node_assignments(world: int, worker_ids: Sequence[str] = (), cuda: bool = True) -> List[RankAssignment]:
    host = os.uname().nodename
    return [RankAssignment(r, r, host, r if cuda else None, tuple(worker_ids)) for r in range(world)]
