"""Controller of long-lived worker groups: requests, health checks, restart with journal replay.

A worker group is a set of rank processes running ``runtime.service`` (one per GPU) that holds a model between
requests. ``WorkerGroupController`` starts the groups through ``LocalWorkerGroupLauncher``, sends each request over
the group's loopback socket and keeps, per group, a JOURNAL of the successful requests that build state from
durable inputs (``build_model``, ``load_*checkpoint``, ``load_weight_version``).

Before every request the group's heartbeats and processes are checked. A group found dead or in error is started
again, at most ``restart_retries`` times, if its state can be rebuilt: that is, if nothing has mutated the model since
the last journalled request (a training step makes a restart unsafe until the next checkpoint or weight-version load
makes it safe again). The new group gets the journal replayed in order before the pending request is sent. A group
that cannot be restarted, and any group whose request fails while in flight, is torn down as a whole (its peers may
sit in a collective that can never complete) and the error names every rank's last heartbeat and log file.
``request_many`` checks all participants first and then runs their requests concurrently (the two ends of a
transfer); if one fails, every participant is aborted.

Reference: RPEG/runtime/semantic_controller.py:226-366 (request paths), :462-538 (health, restart, replay),
:594-636 (journal rules and diagnostics).
"""
from __future__ import annotations

import copy
import json
import socket
from concurrent.futures import ThreadPoolExecutor, as_completed
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

from .errors import RuntimeExecutionError
from .launcher import LocalWorkerGroupLauncher, WorkerLaunch, single_node_assignments
from .service import recv_message, send_message

REPLAYABLE_STATE_OPS = frozenset({"build_model", "load_hf_checkpoint", "load_distributed_checkpoint", "load_weight_version"})


def operation_mutates_model(operation: str) -> bool:
    return operation == "lm_training_step" or operation.endswith("_train_step")


@dataclass(frozen=True)
class WorkerGroupSpec:
    worker_id: str
    world: int = 1
    table: str = "toy"
    backend: str = "gloo"
    master_port: int = 29561
    cuda: bool = False
    env: Dict[str, str] = field(default_factory=dict)
    collective_timeout_s: float = 30.0
    hosts: Tuple[str, ...] = ()          # host of every rank (Slurm launcher); empty: all ranks on this host
    connect_host: Optional[str] = None    # where rank 0's request port is reachable (default: loopback)


@dataclass
class _Journalled:
    operation: str
    node_id: str
    step: int
    payload: Dict[str, Any]
    timeout_s: Optional[float]


class GroupClient:
    """Socket to rank 0 of one worker group."""

    def __init__(self, port: int, connect_timeout_s: float = 10.0, host: str = "127.0.0.1"):
        self.sock = socket.create_connection((host, port), timeout=connect_timeout_s)

    def request(self, operation: str, *, node_id: str, step: int, payload: Optional[Dict[str, Any]] = None,
                timeout_s: Optional[float] = None) -> List[Any]:
        try:
            self.sock.settimeout(timeout_s)
            send_message(self.sock, {"operation": operation, "node_id": node_id, "step": step, "payload": payload or {}})
            reply = recv_message(self.sock)
        except (OSError, ConnectionError, ValueError) as exc:
            raise RuntimeExecutionError(f"no reply to {operation} ({type(exc).__name__}: {exc})") from exc
        if not reply.get("ok"):
            raise RuntimeExecutionError(str(reply.get("error")))
        return reply["results"]

    def close(self) -> None:
        try:
            self.sock.close()
        except OSError:
            pass


@dataclass
class _Managed:
    spec: WorkerGroupSpec
    client: GroupClient
    generation: int


class WorkerGroupController:
    def __init__(self, heartbeat_dir, *, restart_retries: int = 1, log_dir: Optional[str] = None, ready_timeout_s: float = 120.0,
                 stale_after_s: Optional[float] = None, launcher=None):
        """``launcher``: a ``LocalWorkerGroupLauncher`` (default) or a ``SlurmWorkerGroupLauncher`` on the same heartbeat
        directory; with the latter every group is one ``srun`` step and a restart starts a new step."""
        self.launcher = launcher if launcher is not None else LocalWorkerGroupLauncher(heartbeat_dir)
        self.restart_retries = int(restart_retries)
        self.log_dir = log_dir
        self.ready_timeout_s = ready_timeout_s
        self.stale_after_s = stale_after_s
        self._groups: Dict[str, _Managed] = {}
        self._journal: Dict[str, List[_Journalled]] = {}
        self._restart_safe: Dict[str, bool] = {}
        self.restarts: Dict[str, int] = {}
        self._launches: Dict[str, int] = {}

    # ------------------------------------------------------------------------------------------ start / stop
    def start(self, spec: WorkerGroupSpec) -> None:
        if spec.worker_id in self._groups:
            raise RuntimeExecutionError(f"worker group {spec.worker_id} is already running")
        self._groups[spec.worker_id] = self._launch(spec)

    def _launch(self, spec: WorkerGroupSpec) -> _Managed:
        gen = self._launches.get(spec.worker_id, 0)
        self._launches[spec.worker_id] = gen + 1
        # heartbeats of an earlier generation must not be taken for this one's
        for r in range(spec.world):
            self.launcher.store.path(spec.worker_id, r).unlink(missing_ok=True)
        env = dict(spec.env)
        env["RPEG_LAUNCH_GENERATION"] = str(gen)
        self.launcher.launch(WorkerLaunch(spec.worker_id, "rpeg_b200.runtime.service",
                                          ("--table", spec.table, "--backend", spec.backend, "--collective-timeout", str(spec.collective_timeout_s)),
                                          self._assignments(spec),
                                          master_port=spec.master_port + gen, env=env, log_dir=self.log_dir))
        beats = self.launcher.wait_ready(spec.worker_id, self.ready_timeout_s)
        try:
            port = int(json.loads(beats[0].message)["port"])
            client = GroupClient(port, host=spec.connect_host or "127.0.0.1")
        except Exception as exc:
            self.launcher.stop(spec.worker_id, grace_s=1.0)
            raise RuntimeExecutionError(f"{spec.worker_id}: rank 0 came up without a usable request port ({exc})") from exc
        return _Managed(spec, client, gen)

    @staticmethod
    def _assignments(spec: WorkerGroupSpec):
        if not spec.hosts:
            return single_node_assignments(spec.world, (spec.worker_id,), cuda=spec.cuda)
        if len(spec.hosts) != spec.world:
            raise RuntimeExecutionError(f"{spec.worker_id}: {len(spec.hosts)} hosts for {spec.world} ranks")
        from .launcher import RankAssignment
        local: Dict[str, int] = {}
        out = []
        for r, h in enumerate(spec.hosts):
            out.append(RankAssignment(r, local.get(h, 0), h, local.get(h, 0) if spec.cuda else None, (spec.worker_id,)))
            local[h] = local.get(h, 0) + 1
        return out

    def shutdown(self, timeout_s: float = 30.0) -> None:
        for wid, m in list(self._groups.items()):
            try:
                m.client.request("shutdown", node_id="shutdown", step=-1, timeout_s=timeout_s)
                self.launcher.wait_finished(wid, timeout_s)
            except RuntimeExecutionError:
                pass
            m.client.close()
            self.launcher.stop(wid, grace_s=1.0)
        self._groups.clear()

    # ------------------------------------------------------------------------------------------ requests
    def request(self, worker_id: str, operation: str, *, node_id: str, step: int, payload: Optional[Dict[str, Any]] = None,
                timeout_s: Optional[float] = 60.0) -> List[Any]:
        m = self._ensure_healthy_or_restart(self._managed(worker_id), before=f"before {operation}")
        try:
            results = m.client.request(operation, node_id=node_id, step=step, payload=payload, timeout_s=timeout_s)
        except RuntimeExecutionError as exc:
            detail = self.diagnostics(worker_id)
            self._abort(worker_id)
            raise RuntimeExecutionError(f"operation {operation} failed for {worker_id}: {exc}; {detail}; worker group aborted") from exc
        self._record_success(worker_id, _Journalled(operation, node_id, step, copy.deepcopy(payload or {}), timeout_s))
        return results

    def request_many(self, requests: Sequence[Tuple[str, str, str, int, Dict[str, Any], Optional[float]]]) -> Dict[str, List[Any]]:
        """``(worker_id, operation, node_id, step, payload, timeout_s)`` per group, run concurrently. Every participant
        is checked (and restarted if need be) BEFORE either half is sent; one failure aborts all participants."""
        if not requests:
            return {}
        prepared = [(self._ensure_healthy_or_restart(self._managed(w), before=f"before paired {op}"), op, nid, st, pl, to)
                    for w, op, nid, st, pl, to in requests]
        out: Dict[str, List[Any]] = {}
        with ThreadPoolExecutor(max_workers=len(prepared)) as pool:
            futures = {pool.submit(m.client.request, op, node_id=nid, step=st, payload=pl, timeout_s=to): (m, op, nid, st, pl, to)
                       for m, op, nid, st, pl, to in prepared}
            for fut in as_completed(futures):
                m, op, nid, st, pl, to = futures[fut]
                wid = m.spec.worker_id
                try:
                    out[wid] = fut.result()
                    self._record_success(wid, _Journalled(op, nid, st, copy.deepcopy(pl or {}), to))
                except Exception as exc:
                    for other, *_ in prepared:
                        if other.spec.worker_id in self._groups:
                            self._abort(other.spec.worker_id)
                    raise RuntimeExecutionError(f"paired operation {op} failed for {wid}: {exc}; all participants aborted") from exc
        return out

    # ------------------------------------------------------------------------------------------ health, restart, replay
    def _managed(self, worker_id: str) -> _Managed:
        try:
            return self._groups[worker_id]
        except KeyError as exc:
            raise RuntimeExecutionError(f"worker group {worker_id} has not been started (or was aborted)") from exc

    def can_restart(self, worker_id: str) -> bool:
        if self.restart_retries <= 0 or self.restarts.get(worker_id, 0) >= self.restart_retries:
            return False
        return self._restart_safe.get(worker_id, True)

    def _ensure_healthy_or_restart(self, m: _Managed, *, before: str) -> _Managed:
        wid = m.spec.worker_id
        try:
            self.launcher.assert_healthy(wid, self.stale_after_s)
            return m
        except RuntimeExecutionError as exc:
            if not self.can_restart(wid):
                detail = self.diagnostics(wid)
                self._abort(wid)
                why = "its model was changed since the last journalled request" if not self._restart_safe.get(wid, True) else "restarts are exhausted"
                raise RuntimeExecutionError(f"{wid} unhealthy {before}: {exc}; not restarted because {why}; {detail}") from exc
            return self._restart(m, reason=str(exc))

    def _restart(self, m: _Managed, *, reason: str) -> _Managed:
        wid = m.spec.worker_id
        m.client.close()
        self.launcher.stop(wid, grace_s=1.0)
        self._groups.pop(wid, None)
        self.restarts[wid] = self.restarts.get(wid, 0) + 1
        fresh = self._launch(m.spec)
        self._groups[wid] = fresh
        for j in self._journal.get(wid, ()):
            try:
                fresh.client.request(j.operation, node_id=j.node_id, step=j.step, payload=copy.deepcopy(j.payload), timeout_s=j.timeout_s)
            except RuntimeExecutionError as exc:
                detail = self.diagnostics(wid)
                self._abort(wid)
                raise RuntimeExecutionError(f"{wid}: replay of {j.operation} ({j.node_id}) failed after restart for '{reason}': {exc}; {detail}") from exc
        return fresh

    def _record_success(self, worker_id: str, j: _Journalled) -> None:
        if j.operation in REPLAYABLE_STATE_OPS:
            journal = self._journal.setdefault(worker_id, [])
            if j.operation == "build_model":
                journal.clear()                      # a rebuilt model supersedes everything before it
            elif journal and journal[-1].operation == j.operation and j.operation.startswith("load_"):
                journal.pop()                        # a newer load of the same kind replaces the older one
            journal.append(j)
            self._restart_safe[worker_id] = True
        elif operation_mutates_model(j.operation):
            self._restart_safe[worker_id] = False

    def journal(self, worker_id: str) -> List[Tuple[str, str]]:
        return [(j.operation, j.node_id) for j in self._journal.get(worker_id, ())]

    def _abort(self, worker_id: str) -> None:
        m = self._groups.pop(worker_id, None)
        if m is not None:
            m.client.close()
        self.launcher.stop(worker_id, grace_s=1.0)

    def diagnostics(self, worker_id: str) -> str:
        m = self._groups.get(worker_id)
        world = m.spec.world if m is not None else 0
        beats = self.launcher.store.read_group(worker_id, world)
        ranks = ", ".join(f"rank {r}: missing" if hb is None else f"rank {r} state={hb.state}" + (f" message={hb.message!r}" if hb.message else "")
                          for r, hb in enumerate(beats))
        logs = f", logs={self.log_dir}/{worker_id}.rank*.log" if self.log_dir else ""
        return f"heartbeats=[{ranks}]{logs}"
