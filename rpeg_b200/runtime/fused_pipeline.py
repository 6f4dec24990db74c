"""Offline scheduler for intra-stage actor/critic training fusion.

Two pipeline-parallel models share the same GPUs: the actor runs its stages in device order, the
critic in reverse order, and their forward/backward microtasks are interleaved on every device by a
precomputed instruction stream. The planner uses the schedule's makespan and peak live activations;
the runtime replays ``local_instructions`` on two CUDA streams of one process per GPU.

Behaviour follows the reference (RPEG/runtime/fused_pipeline.py:24-939):
  * tasks ``model:F{mb}:s{stage}`` / ``model:B{mb}:s{stage}``; per microbatch the chain F(s0..)
    then B(..s0); per (model, stage) all forwards in microbatch order, then all backwards;
  * deterministic list scheduling, one instruction stream per physical stage, with ten priority
    rules; ``portfolio`` builds all of them, keeps the valid ones and returns the one with the
    smallest (makespan, max peak activation, total peak activation, device order);
  * validation covers dependencies, per-device exclusivity, activation accounting and a simulation
    of blocking point-to-point rendezvous that proves the instruction streams cannot deadlock.
Schema id of the serialised form: ``rpeg.fused_pipeline_schedule.v1``.
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass
from functools import lru_cache
from typing import Dict, Iterable, List, Mapping, Optional, Tuple

SCHEMA = "rpeg.fused_pipeline_schedule.v1"
PRIORITY_MODES = (
    "greedy_backward_work", "critical_path", "forward_wave", "microbatch_wave",
    "model_serial", "model_serial_reverse",
    "phase_af_cf_ab_cb", "phase_af_cf_cb_ab", "phase_cf_af_ab_cb", "phase_cf_af_cb_ab",
)
_BARRIER_ORDERS = {
    "model_serial": ((0, "F"), (0, "B"), (1, "F"), (1, "B")),
    "model_serial_reverse": ((1, "F"), (1, "B"), (0, "F"), (0, "B")),
    "phase_af_cf_ab_cb": ((0, "F"), (1, "F"), (0, "B"), (1, "B")),
    "phase_af_cf_cb_ab": ((0, "F"), (1, "F"), (1, "B"), (0, "B")),
    "phase_cf_af_ab_cb": ((1, "F"), (0, "F"), (0, "B"), (1, "B")),
    "phase_cf_af_cb_ab": ((1, "F"), (0, "F"), (1, "B"), (0, "B")),
}


class FusedPipelineError(ValueError):
    pass


@dataclass(frozen=True, order=True)
class FusedPipelineTask:
    model: str
    microbatch: int
    phase: str
    stage: int
    device_stage: int
    duration_s: float
    activation_bytes: int

    def __post_init__(self) -> None:
        if not self.model or self.phase not in ("F", "B"):
            raise FusedPipelineError(f"bad fused pipeline task {self.model!r}/{self.phase!r}")
        if min(self.microbatch, self.stage, self.device_stage, self.activation_bytes) < 0 or self.duration_s <= 0.0:
            raise FusedPipelineError("fused pipeline task indices/bytes must be >= 0 and duration > 0")

    @property
    def task_id(self) -> str:
        return f"{self.model}:{self.phase}{self.microbatch}:s{self.stage}"

    def to_dict(self) -> dict:
        return {"task_id": self.task_id, "model": self.model, "microbatch": self.microbatch, "phase": self.phase,
                "stage": self.stage, "device_stage": self.device_stage, "duration_s": self.duration_s,
                "activation_bytes": self.activation_bytes}


@dataclass(frozen=True)
class FusedPipelineModel:
    name: str
    pipeline_stages: int
    microbatches: int
    forward_s: Tuple[float, ...]
    backward_s: Tuple[float, ...]
    activation_bytes: Tuple[int, ...]
    reverse: bool = False

    @classmethod
    def uniform(cls, name: str, *, pipeline_stages: int, microbatches: int, forward_s: float, backward_s: float,
                activation_bytes: int, reverse: bool = False) -> "FusedPipelineModel":
        p = int(pipeline_stages)
        return cls(name, p, int(microbatches), (float(forward_s),) * p, (float(backward_s),) * p,
                   (int(activation_bytes),) * p, bool(reverse))

    def __post_init__(self) -> None:
        if not self.name:
            raise FusedPipelineError("fused pipeline model needs a name")
        if self.pipeline_stages <= 1:
            raise FusedPipelineError("intra-stage fusion requires pipeline_stages > 1")
        if self.microbatches < self.pipeline_stages:
            raise FusedPipelineError(f"{self.name}: microbatches={self.microbatches} must be >= pipeline_stages={self.pipeline_stages}")
        for label, vals in (("forward_s", self.forward_s), ("backward_s", self.backward_s), ("activation_bytes", self.activation_bytes)):
            if len(vals) != self.pipeline_stages:
                raise FusedPipelineError(f"{self.name}: {label} needs {self.pipeline_stages} entries")
        if any(v <= 0.0 for v in self.forward_s + self.backward_s) or any(v < 0 for v in self.activation_bytes):
            raise FusedPipelineError(f"{self.name}: durations must be > 0 and activation bytes >= 0")

    def device_stage(self, logical_stage: int) -> int:
        if not 0 <= logical_stage < self.pipeline_stages:
            raise FusedPipelineError(f"{self.name}: stage {logical_stage} outside the pipeline")
        return self.pipeline_stages - 1 - logical_stage if self.reverse else logical_stage

    def to_dict(self) -> dict:
        return {"name": self.name, "pipeline_stages": self.pipeline_stages, "microbatches": self.microbatches,
                "forward_s": list(self.forward_s), "backward_s": list(self.backward_s),
                "activation_bytes": list(self.activation_bytes), "reverse": self.reverse}


@dataclass(frozen=True)
class FusedPipelineSchedule:
    models: Tuple[FusedPipelineModel, ...]
    tasks: Tuple[FusedPipelineTask, ...]
    dependencies: Tuple[Tuple[str, str], ...]
    device_order: Tuple[Tuple[str, ...], ...]
    start_s: Tuple[Tuple[str, float], ...]
    finish_s: Tuple[Tuple[str, float], ...]
    peak_activation_bytes: Tuple[int, ...]
    makespan_s: float
    optimizer: str = "greedy_backward_work"
    optimizer_candidates: int = 1
    baseline_makespan_s: Optional[float] = None

    @property
    def schedule_hash(self) -> str:
        body = json.dumps(self.to_dict(include_timings=False), sort_keys=True, separators=(",", ":"))
        return hashlib.sha256(body.encode()).hexdigest()

    def to_dict(self, *, include_timings: bool = True) -> dict:
        out = {"schema_version": SCHEMA, "models": [m.to_dict() for m in self.models],
               "tasks": [t.to_dict() for t in self.tasks], "dependencies": [list(d) for d in self.dependencies],
               "device_order": [list(o) for o in self.device_order], "optimizer": self.optimizer}
        if include_timings:
            out.update(start_s=dict(self.start_s), finish_s=dict(self.finish_s),
                       peak_activation_bytes=list(self.peak_activation_bytes), makespan_s=self.makespan_s,
                       optimizer_candidates=self.optimizer_candidates, baseline_makespan_s=self.baseline_makespan_s,
                       schedule_hash=self.schedule_hash)
        return out

    @classmethod
    def from_dict(cls, raw: Mapping) -> "FusedPipelineSchedule":
        if raw.get("schema_version") != SCHEMA:
            raise FusedPipelineError(f"expected schema {SCHEMA}, got {raw.get('schema_version')!r}")
        models = tuple(FusedPipelineModel(m["name"], int(m["pipeline_stages"]), int(m["microbatches"]),
                                          tuple(map(float, m["forward_s"])), tuple(map(float, m["backward_s"])),
                                          tuple(map(int, m["activation_bytes"])), bool(m.get("reverse", False)))
                       for m in raw["models"])
        tasks = tuple(FusedPipelineTask(t["model"], int(t["microbatch"]), t["phase"], int(t["stage"]),
                                        int(t["device_stage"]), float(t["duration_s"]), int(t["activation_bytes"]))
                      for t in raw["tasks"])
        sched = cls(models, tasks, tuple((a, b) for a, b in raw["dependencies"]),
                    tuple(tuple(o) for o in raw["device_order"]), tuple(sorted(raw.get("start_s", {}).items())),
                    tuple(sorted(raw.get("finish_s", {}).items())), tuple(raw.get("peak_activation_bytes", ())),
                    float(raw.get("makespan_s", 0.0)), raw.get("optimizer", "greedy_backward_work"),
                    int(raw.get("optimizer_candidates", 1)), raw.get("baseline_makespan_s"))
        want = raw.get("schedule_hash")
        if want is not None and want != sched.schedule_hash:
            raise FusedPipelineError("fused pipeline schedule hash mismatch")
        return sched

    def local_instructions(self, model: str, device_stage: int) -> Tuple[dict, ...]:
        """Instruction stream of ``model`` on one physical stage, each with the task that must have
        finished on this device before it (``after``), whichever model that task belongs to."""
        by_id = {t.task_id: t for t in self.tasks}
        order = self.device_order[device_stage]
        out = []
        for i, tid in enumerate(order):
            t = by_id[tid]
            if t.model == model:
                out.append({**t.to_dict(), "device_index": i, "after": order[i - 1] if i else None})
        return tuple(out)


def _build_tasks(models: Tuple[FusedPipelineModel, ...]):
    tasks: Dict[str, FusedPipelineTask] = {}
    deps = set()
    for m in models:
        for mb in range(m.microbatches):
            chain = []
            for phase, stages in (("F", range(m.pipeline_stages)), ("B", reversed(range(m.pipeline_stages)))):
                for s in stages:
                    dur = m.forward_s[s] if phase == "F" else m.backward_s[s]
                    t = FusedPipelineTask(m.name, mb, phase, s, m.device_stage(s), float(dur), int(m.activation_bytes[s]))
                    tasks[t.task_id] = t
                    chain.append(t.task_id)
            deps.update(zip(chain, chain[1:]))
        # forward wave, then backward wave, on every logical stage: a blocking send of one phase can
        # then never face a peer that is waiting in the other phase
        for s in range(m.pipeline_stages):
            wave = [f"{m.name}:F{mb}:s{s}" for mb in range(m.microbatches)] + [f"{m.name}:B{mb}:s{s}" for mb in range(m.microbatches)]
            deps.update(zip(wave, wave[1:]))
    return tasks, deps


def _remaining_paths(tasks, succ, pred) -> Dict[str, float]:
    indeg = {t: len(pred[t]) for t in tasks}
    order, queue = [], sorted(t for t, c in indeg.items() if c == 0)
    head = 0
    while head < len(queue):
        u = queue[head]
        head += 1
        order.append(u)
        for w in sorted(succ[u]):
            indeg[w] -= 1
            if indeg[w] == 0:
                queue.append(w)
    if len(order) != len(tasks):
        raise FusedPipelineError("fused pipeline dependency cycle")
    rem: Dict[str, float] = {}
    for t in reversed(order):
        rem[t] = tasks[t].duration_s + max((rem[w] for w in succ[t]), default=0.0)
    return rem


def _peak_activation(tasks: Mapping[str, FusedPipelineTask], finish: Mapping[str, float], n_dev: int) -> List[int]:
    """Forward finishes allocate, backward finishes release; allocations first on timestamp ties."""
    events: List[list] = [[] for _ in range(n_dev)]
    for tid, t in tasks.items():
        events[t.device_stage].append((finish[tid], 0 if t.phase == "F" else 1, tid, t.activation_bytes if t.phase == "F" else -t.activation_bytes))
    peaks = [0] * n_dev
    for d, evs in enumerate(events):
        live = 0
        for _, _, _, delta in sorted(evs):
            live += delta
            if live < 0:
                raise FusedPipelineError(f"fused pipeline stage {d} releases an activation before its forward")
            peaks[d] = max(peaks[d], live)
        if live != 0:
            raise FusedPipelineError(f"fused pipeline stage {d} leaves {live} activation bytes live")
    return peaks


def _capacities(cap, n_dev):
    if cap is None:
        return None
    if isinstance(cap, int):
        return (cap,) * n_dev
    cap = tuple(int(c) for c in cap)
    if len(cap) != n_dev:
        raise FusedPipelineError(f"activation capacity needs {n_dev} entries")
    return cap


def simulate_blocking_p2p(schedule: FusedPipelineSchedule) -> None:
    """Run the instruction streams as one sequential process per (model, stage) whose sends block
    until the peer posts the matching receive; raises if the streams cannot all finish."""
    tasks = {t.task_id: t for t in schedule.tasks}
    models = {m.name: m for m in schedule.models}
    procs = {(m.name, s): tuple(t for t in schedule.device_order[m.device_stage(s)] if tasks[t].model == m.name)
             for m in schedule.models for s in range(m.pipeline_stages)}
    dev_pred = {tid: (order[i - 1] if i else None) for order in schedule.device_order for i, tid in enumerate(order)}
    idx = {p: 0 for p in procs}
    state = {p: "new" for p in procs}
    computed = set()
    sends: Dict[tuple, tuple] = {}
    recvs: Dict[tuple, tuple] = {}

    def has_recv(t):
        return (t.phase == "F" and t.stage > 0) or (t.phase == "B" and t.stage < models[t.model].pipeline_stages - 1)

    def has_send(t):
        return (t.phase == "F" and t.stage < models[t.model].pipeline_stages - 1) or (t.phase == "B" and t.stage > 0)

    def chan(t, sending: bool):
        if sending:
            link = t.stage if t.phase == "F" else t.stage - 1
        else:
            link = t.stage - 1 if t.phase == "F" else t.stage
        return (t.model, t.phase, t.microbatch, link)

    def computed_now(p, t):
        computed.add(t.task_id)
        if has_send(t):
            c = chan(t, True)
            if c in sends:
                raise FusedPipelineError(f"duplicate blocking send on {c}")
            state[p] = "send"
            sends[c] = p
        else:
            idx[p] += 1
            state[p] = "new"

    for _ in range(len(tasks) * 8 + 1):
        progress = False
        for p in sorted(procs):
            seq = procs[p]
            if idx[p] >= len(seq) or state[p] != "new":
                continue
            t = tasks[seq[idx[p]]]
            before = dev_pred[t.task_id]
            if before is not None and before not in computed:
                continue
            if has_recv(t):
                c = chan(t, False)
                if c in recvs:
                    raise FusedPipelineError(f"duplicate blocking recv on {c}")
                state[p] = "recv"
                recvs[c] = p
            else:
                computed_now(p, t)
            progress = True
        for c in sorted(set(sends) & set(recvs)):
            sender, receiver = sends.pop(c), recvs.pop(c)
            rt = tasks[procs[receiver][idx[receiver]]]
            idx[sender] += 1
            state[sender] = "new"
            computed_now(receiver, rt)
            progress = True
        if all(idx[p] >= len(seq) for p, seq in procs.items()):
            return
        if not progress:
            stuck = [f"{p[0]}:s{p[1]}:{state[p]}:{procs[p][idx[p]]}" for p in sorted(procs) if idx[p] < len(procs[p])]
            raise FusedPipelineError(f"fused pipeline blocking P2P execution deadlocks: {stuck[:16]}")
    raise FusedPipelineError("fused pipeline blocking P2P validation did not converge")


def validate_fused_pipeline_schedule(schedule: FusedPipelineSchedule, *, activation_capacity_bytes=None) -> None:
    tasks = {t.task_id: t for t in schedule.tasks}
    start, finish = dict(schedule.start_s), dict(schedule.finish_s)
    if set(start) != set(tasks) or set(finish) != set(tasks):
        raise FusedPipelineError("fused pipeline schedule does not time every task exactly once")
    want_tasks, want_deps = _build_tasks(schedule.models)
    if set(want_tasks) != set(tasks) or set(want_deps) != set(schedule.dependencies):
        raise FusedPipelineError("fused pipeline task or dependency set does not match its models")
    eps = 1e-12
    for a, b in schedule.dependencies:
        if finish[a] > start[b] + eps:
            raise FusedPipelineError(f"dependency {a} -> {b} violated")
    n_dev = len(schedule.device_order)
    seen = set()
    for d, order in enumerate(schedule.device_order):
        t_prev = 0.0
        for tid in order:
            if tid in seen or tasks[tid].device_stage != d:
                raise FusedPipelineError(f"task {tid} misplaced in device order")
            seen.add(tid)
            if start[tid] + eps < t_prev:
                raise FusedPipelineError(f"tasks overlap on stage {d} at {tid}")
            if abs(finish[tid] - start[tid] - tasks[tid].duration_s) > 1e-9 * max(1.0, tasks[tid].duration_s):
                raise FusedPipelineError(f"task {tid} has the wrong duration")
            t_prev = finish[tid]
    if seen != set(tasks):
        raise FusedPipelineError("device order does not cover every task")
    peaks = _peak_activation(tasks, finish, n_dev)
    if tuple(peaks) != tuple(schedule.peak_activation_bytes):
        raise FusedPipelineError("peak activation bytes do not match the timings")
    caps = _capacities(activation_capacity_bytes, n_dev)
    if caps is not None:
        bad = [(d, p, caps[d]) for d, p in enumerate(peaks) if p > caps[d]]
        if bad:
            raise FusedPipelineError("fused pipeline activation memory exceeds capacity: " +
                                     ", ".join(f"stage {d}: peak={p} capacity={c}" for d, p, c in bad))
    simulate_blocking_p2p(schedule)


def _list_schedule(models: Tuple[FusedPipelineModel, ...], mode: str, cap) -> FusedPipelineSchedule:
    tasks, deps = _build_tasks(models)
    succ = {t: set() for t in tasks}
    pred = {t: set() for t in tasks}
    for a, b in deps:
        succ[a].add(b)
        pred[b].add(a)
    rem = _remaining_paths(tasks, succ, pred)
    work = {m.name: m.microbatches * sum(m.forward_s + m.backward_s) for m in models}
    n_dev = models[0].pipeline_stages
    left = {t: len(pred[t]) for t in tasks}
    pred_fin = {t: 0.0 for t in tasks}
    dev_free = [0.0] * n_dev
    order: List[List[str]] = [[] for _ in range(n_dev)]
    start: Dict[str, float] = {}
    finish: Dict[str, float] = {}
    ready = {t for t, c in left.items() if c == 0}
    group = ({(models[i].name, ph): g for g, (i, ph) in enumerate(_BARRIER_ORDERS[mode])} if mode in _BARRIER_ORDERS else None)

    def key(tid: str):
        t = tasks[tid]
        est = max(pred_fin[tid], dev_free[t.device_stage])
        tail = (t.model, t.stage, tid)
        if group is not None:
            return (group[(t.model, t.phase)], est, t.microbatch, *tail)
        if mode == "critical_path":
            return (est, -rem[tid], 0 if t.phase == "B" else 1, -work[t.model], t.microbatch, *tail)
        if mode == "forward_wave":
            return (est, 0 if t.phase == "F" else 1, t.microbatch, -rem[tid], *tail)
        if mode == "microbatch_wave":
            return (est, t.microbatch, 0 if t.phase == "B" else 1, -rem[tid], *tail)
        return (est, 0 if t.phase == "B" else 1, -work[t.model], t.microbatch, *tail)  # greedy_backward_work

    while ready:
        tid = min(ready, key=key)
        ready.remove(tid)
        t = tasks[tid]
        s = max(pred_fin[tid], dev_free[t.device_stage])
        start[tid], finish[tid] = s, s + t.duration_s
        dev_free[t.device_stage] = finish[tid]
        order[t.device_stage].append(tid)
        for w in succ[tid]:
            left[w] -= 1
            pred_fin[w] = max(pred_fin[w], finish[tid])
            if left[w] == 0:
                ready.add(w)
    if len(finish) != len(tasks):
        raise FusedPipelineError("fused pipeline dependency cycle")
    peaks = _peak_activation(tasks, finish, n_dev)
    sched = FusedPipelineSchedule(models, tuple(sorted(tasks.values(), key=lambda t: t.task_id)), tuple(sorted(deps)),
                                  tuple(tuple(o) for o in order), tuple(sorted(start.items())),
                                  tuple(sorted(finish.items())), tuple(peaks), max(finish.values(), default=0.0), mode, 1, None)
    validate_fused_pipeline_schedule(sched, activation_capacity_bytes=cap)
    return sched


@lru_cache(maxsize=4096)
def _build_cached(models: Tuple[FusedPipelineModel, ...], cap, optimization: str) -> FusedPipelineSchedule:
    if len(models) != 2:
        raise FusedPipelineError("actor/critic intra-stage fusion needs exactly two models")
    if models[0].name == models[1].name:
        raise FusedPipelineError("fused pipeline model names must be unique")
    if models[0].pipeline_stages != models[1].pipeline_stages:
        raise FusedPipelineError("fused models must have the same number of pipeline stages")
    if models[0].reverse == models[1].reverse:
        raise FusedPipelineError("fused models must run in opposite directions")
    if optimization != "portfolio":
        if optimization not in PRIORITY_MODES:
            raise FusedPipelineError(f"unsupported fused pipeline optimization {optimization!r}")
        return _list_schedule(models, optimization, cap)
    valid, errors, baseline = [], [], None
    for mode in PRIORITY_MODES:
        try:
            s = _list_schedule(models, mode, cap)
        except FusedPipelineError as exc:
            errors.append(f"{mode}: {exc}")
            continue
        valid.append(s)
        if mode == "greedy_backward_work":
            baseline = s.makespan_s
    if not valid:
        raise FusedPipelineError("no valid fused pipeline schedule: " + "; ".join(errors))
    best = min(valid, key=lambda s: (s.makespan_s, max(s.peak_activation_bytes), sum(s.peak_activation_bytes), s.device_order))
    return FusedPipelineSchedule(best.models, best.tasks, best.dependencies, best.device_order, best.start_s, best.finish_s,
                                 best.peak_activation_bytes, best.makespan_s, "deterministic_blocking_safe_portfolio_v2",
                                 len(valid), baseline)


def build_fused_pipeline_schedule(models: Iterable[FusedPipelineModel], *, activation_capacity_bytes=None,
                                  optimization: str = "portfolio") -> FusedPipelineSchedule:
    cap = activation_capacity_bytes
    if cap is not None and not isinstance(cap, int):
        cap = tuple(int(c) for c in cap)
    return _build_cached(tuple(models), cap, optimization)


def peak_activation_bytes(schedule: FusedPipelineSchedule) -> Tuple[int, ...]:
    return tuple(schedule.peak_activation_bytes)
