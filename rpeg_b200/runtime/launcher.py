"""Launching the rank processes of a job on one node and tearing them down.

One process per GPU. ``LocalWorkerGroupLauncher`` starts ``world`` Python processes in a session of
their own (so the whole group can be signalled by process-group id and nothing else is touched),
gives each its rendezvous environment (loopback address, one port per job) and the JSON rank
assignment, waits for ``ready`` heartbeats and stops the group with SIGTERM followed by SIGKILL
after a grace period. ``torchrun_command`` renders the equivalent ``torch.distributed.run`` line for
a user who launches by hand. ``SlurmWorkerGroupLauncher`` starts the same rank processes as tasks of ONE ``srun`` step
inside an existing allocation (one group, or a pool of several groups that must share a step): it writes a manifest
that tells every task of the step which rank of which group it is (``runtime/pool_entry.py``), pads hosts with fewer
ranks with idle tasks so that the step is uniform, and ends the step through a stop file and SIGTERM.
Reference: RPEG/runtime/launcher.py:27-211 (local launcher), :212-531 (Slurm launcher: srun --overlap, shared-step pool
and its manifest, stop file). `runtime.job_plan --emit-sbatch` writes the batch file for whole SPMD jobs
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


# ------------------------------------------------------------------------------------------------ Slurm
@dataclass
class SlurmOptions:
    partition: Optional[str] = None
    account: Optional[str] = None
    time_limit: Optional[str] = None
    container_image: Optional[str] = None
    mpi: str = "none"
    srun: str = "srun"
    extra: Sequence[str] = ()


class SlurmWorkerGroupLauncher:
    """Worker groups as tasks of one ``srun --overlap`` step each (``launch``), or several groups in ONE step
    (``launch_pool``: interconnect credentials that are scoped to a step make separately started steps unable to talk to
    each other). Same interface as ``LocalWorkerGroupLauncher`` where a controller needs it."""

    def __init__(self, heartbeat_dir, work_dir, options: Optional[SlurmOptions] = None, poll_s: float = 0.05,
                 require_allocation: bool = True):
        self.heartbeat_dir = str(heartbeat_dir)
        self.work_dir = Path(work_dir)
        self.options = options or SlurmOptions()
        self.store = HeartbeatStore(heartbeat_dir)
        self.control = ControlPlane(self.store, poll_s)
        self.require_allocation = require_allocation
        self.steps: Dict[str, subprocess.Popen] = {}          # step name -> srun process
        self.step_of: Dict[str, str] = {}                     # group id -> step name
        self.launches: Dict[str, WorkerLaunch] = {}
        self.stop_paths: Dict[str, Path] = {}

    # -- what would run
    def manifest(self, step: str, launches: Sequence[WorkerLaunch]) -> Dict:
        """Tasks of the step, host by host: every host gets as many slots as the fullest one (idle fillers behind its
        ranks), because a step has one task count per node."""
        hosts: Dict[str, List[str]] = {}
        per_host: Dict[str, List] = {}
        for launch in launches:
            if not launch.assignments:
                raise RuntimeExecutionError(f"worker group {launch.group_id} has no ranks")
            for a in launch.assignments:
                per_host.setdefault(a.hostname.split(".", 1)[0], []).append((launch, a))
        width = max(len(v) for v in per_host.values())
        tasks: Dict[str, Dict] = {}
        root = self.work_dir / step
        for hi, (host, ranks) in enumerate(per_host.items()):
            hosts[host] = []
            for slot in range(width):
                tid = str(hi * width + slot)
                hosts[host].append(tid)
                if slot >= len(ranks):
                    tasks[tid] = {"idle": True, "hostname": host}
                    continue
                launch, a = ranks[slot]
                env = {k: v for k, v in rank_environment(launch, a, self.heartbeat_dir).items()
                       if k in launch.env or k.startswith(("RPEG_", "MASTER_")) or k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "PYTHONPATH")}
                # the rendezvous address is the host of the group's rank 0, not the loopback of a single node
                first = launch.assignments[0].hostname
                if len({x.hostname for x in launch.assignments}) > 1:
                    env["MASTER_ADDR"] = first
                tasks[tid] = {"idle": False, "hostname": host, "group_id": launch.group_id, "rank": a.rank, "module": launch.module,
                              "argv": list(launch.args), "env": env,
                              "log": str(Path(launch.log_dir) / f"{launch.group_id}.rank{a.rank}.log") if launch.log_dir else None}
        return {"schema": "rpeg.worker_pool.v1", "step": step, "stop_path": str(root / "stop"), "hosts": hosts, "tasks": tasks,
                "slots_per_host": width}

    def srun_command(self, manifest: Dict, manifest_path: Path) -> List[str]:
        o, hosts = self.options, list(manifest["hosts"])
        width = int(manifest["slots_per_host"])
        cmd = [o.srun, "--overlap", "--nodes", str(len(hosts)), "--ntasks", str(len(hosts) * width), "--ntasks-per-node", str(width),
               "--nodelist", ",".join(hosts), "--distribution", "block:block", "--export", "ALL", "--mpi", o.mpi, "--kill-on-bad-exit=1"]
        for flag, value in (("--partition", o.partition), ("--account", o.account), ("--time", o.time_limit),
                            ("--container-image", o.container_image)):
            if value:
                cmd += [flag, str(value)]
        cmd += list(o.extra)
        return cmd + [sys.executable, "-m", "rpeg_b200.runtime.pool_entry", "--manifest", str(manifest_path)]

    # -- launching
    def launch(self, launch: WorkerLaunch) -> None:
        self.launch_pool([launch], step=launch.group_id)

    def launch_pool(self, launches: Sequence[WorkerLaunch], step: str = "pool") -> None:
        if self.require_allocation and not os.environ.get("SLURM_JOB_ID"):
            raise RuntimeExecutionError("the Slurm launcher must run inside an existing allocation (SLURM_JOB_ID is not set)")
        if step in self.steps and self.steps[step].poll() is None:
            raise RuntimeExecutionError(f"step {step} is already running")
        for launch in launches:
            if launch.group_id in self.step_of:
                raise RuntimeExecutionError(f"worker group {launch.group_id} is already running")
            for a in launch.assignments:                    # heartbeats of an earlier incarnation must not be taken for this one's
                self.store.path(launch.group_id, a.rank).unlink(missing_ok=True)
        man = self.manifest(step, launches)
        root = self.work_dir / step
        root.mkdir(parents=True, exist_ok=True)
        Path(man["stop_path"]).unlink(missing_ok=True)
        path = root / "launch_manifest.json"
        path.write_text(json.dumps(man, indent=1))
        env = dict(os.environ)
        env["PYTHONPATH"] = str(Path(__file__).resolve().parents[2]) + (os.pathsep + env["PYTHONPATH"] if env.get("PYTHONPATH") else "")
        out = open(root / "srun.log", "w")
        self.steps[step] = subprocess.Popen(self.srun_command(man, path), env=env, stdout=out, stderr=subprocess.STDOUT,
                                            start_new_session=True)
        out.close()
        self.stop_paths[step] = Path(man["stop_path"])
        for launch in launches:
            self.step_of[launch.group_id] = step
            self.launches[launch.group_id] = launch

    # -- the interface a controller uses
    def alive(self, group_id: str):
        proc = self.steps[self.step_of[group_id]]
        return lambda rank: proc.poll() is None        # one process stands for the step; ranks report through heartbeats

    def wait_ready(self, group_id: str, timeout_s: float = 120.0):
        try:
            return self.control.wait_for_state(group_id, self.launches[group_id].world, ("ready", "running", "finished"), timeout_s,
                                               alive=self.alive(group_id))
        except RuntimeExecutionError:
            self.stop(group_id, grace_s=1.0)
            raise

    def assert_healthy(self, group_id: str, stale_after_s: Optional[float] = None) -> None:
        self.control.assert_healthy(group_id, self.launches[group_id].world, alive=self.alive(group_id), stale_after_s=stale_after_s)

    def wait_finished(self, group_id: str, timeout_s: float) -> List[int]:
        """Until every rank of the group reported ``finished`` (the step itself may go on: other groups, idle tasks)."""
        self.control.wait_for_state(group_id, self.launches[group_id].world, ("finished",), timeout_s)
        return [0] * self.launches[group_id].world

    def stop(self, group_id: str, grace_s: float = 5.0) -> None:
        """Ends the STEP the group runs in (a step cannot lose single tasks): stop file for the idle tasks, SIGTERM to srun
        (which forwards it), SIGKILL after the grace period."""
        step = self.step_of.get(group_id)
        if step is None:
            return
        self.stop_step(step, grace_s)

    def stop_step(self, step: str, grace_s: float = 5.0) -> None:
        proc = self.steps.pop(step, None)
        stop_path = self.stop_paths.pop(step, None)
        if stop_path is not None:
            stop_path.parent.mkdir(parents=True, exist_ok=True)
            stop_path.write_text("stop\n")
        for g in [g for g, s in self.step_of.items() if s == step]:
            self.step_of.pop(g, None)
            self.launches.pop(g, None)
        if proc is None:
            return
        for sig, wait in ((None, min(grace_s, 2.0)), (signal.SIGTERM, grace_s), (signal.SIGKILL, 1.0)):
            if proc.poll() is not None:
                break
            if sig is not None:
                try:
                    os.killpg(proc.pid, sig)
                except (ProcessLookupError, PermissionError):
                    pass
            deadline = time.monotonic() + wait
            while time.monotonic() < deadline and proc.poll() is None:
                time.sleep(0.02)

    def stop_all(self) -> None:
        for step in list(self.steps):
            self.stop_step(step)

