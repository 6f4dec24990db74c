"""Oracle for any backend: check a JSONL runtime trace against the compiled plan and graph.

Checks (reference: RPEG/runtime/verification.py:144-895):
  coverage      every graph node has exactly one successful start/finish pair (per attempt), no
                unknown nodes, a single run id;
  ordering      ``finish(dep) <= start(node)`` for every dependency;
  exclusivity   two nodes holding a common resource key never overlap in time, except members of one
                fused launch (same ``batch_scheduled_nodes``);
  steps         the traced step of a node equals its logical step;
  versions      serving operators of trainable models consumed ``max(0, step-1-tau)`` and report the
                right shadow flag; training produced versions 1, 2, ... in order per model;
  quantiles     split nodes carry the planner's ``n_seqs``/phase/offset/part counters; generation
                phases report no forced completions; emitted rows of all phases of a step sum to B*K
                when the backend reports them;
  transfers     payload bytes equal the planned payload;
  recovery      ``replay`` / ``recover`` events are consistent with the attempts seen.
Returns a report dict; ``raise_on_error`` turns violations into ``RuntimeExecutionError``.
"""
from __future__ import annotations

from typing import Any, Dict, Iterable, List, Optional, Sequence

from ..passes.lower import ExecNodeType
from .errors import RuntimeExecutionError
from .executor import TRAINABLE_NAMES, model_name
from .graph import RuntimeGraph, suffix_node_ids
from .weight_versions import consumer_weight_version, uses_shadow_copies

LIFECYCLE_NODES = ("runtime.workers.start", "runtime.workers.initialize", "runtime.weights.publish_initial",
                   "runtime.transports.prewarm", "runtime.checkpoint.save", "runtime.checkpoint.restore")
_EPS = 1e-9


def _tau_by_name(compiled) -> Dict[str, int]:
    out = {}
    if compiled is not None:
        for m, t in compiled.config.rpeg.tau.items():
            out[model_name(m.value)] = int(t)
    return out


def verify_runtime_trace(compiled, graph: RuntimeGraph, events: Sequence[dict], *, raise_on_error: bool = True,
                         completed_before: Iterable[str] = ()) -> Dict[str, Any]:
    """``completed_before``: nodes satisfied by a restored checkpoint (absent from a suffix run)."""
    errors: List[str] = []
    warn: List[str] = []
    skip = set(completed_before)
    run_ids = {e.get("run_id") for e in events}
    if len(run_ids) > 1:
        errors.append(f"trace mixes run ids {sorted(map(str, run_ids))}")
    starts: Dict[str, dict] = {}
    finishes: Dict[str, dict] = {}
    attempts = {"replay": 0, "recover": 0}
    failed: List[str] = []
    restored_steps: List[int] = []
    for e in events:
        nid, ev = e.get("node_id"), e.get("event")
        if ev in attempts:
            attempts[ev] += 1
            if ev == "replay":
                # a failed attempt leaves starts without finishes behind
                starts = {k: v for k, v in starts.items() if k in finishes}
            else:
                # nodes after the restored step run again in the next attempt: forget their first execution
                restored = int((e.get("counters") or {}).get("restored_step", 0))
                for k in suffix_node_ids(graph, restored):
                    finishes.pop(k, None)
                    starts.pop(k, None)
                restored_steps.append(restored)
            continue
        if nid in LIFECYCLE_NODES:
            continue
        if nid not in graph.nodes:
            errors.append(f"trace names unknown node {nid}")
            continue
        if ev == "start":
            if nid in starts and nid in finishes:
                errors.append(f"{nid} started again after finishing")
            starts[nid] = e
        elif ev == "finish":
            if e.get("status") != "ok":
                failed.append(nid)
                starts.pop(nid, None)
                continue
            if nid not in starts:
                errors.append(f"{nid} finished without a start")
            if nid in finishes:
                errors.append(f"{nid} finished twice")
            finishes[nid] = e
    for nid in graph.nodes:
        if nid in skip:
            continue
        if nid not in starts or nid not in finishes:
            errors.append(f"{nid} has no successful start/finish pair")
    if failed and attempts["replay"] == 0:
        errors.append(f"nodes failed without a replay attempt: {sorted(set(failed))[:10]}")
    t0 = {n: float(starts[n]["timestamp"]) for n in starts if n in finishes}
    t1 = {n: float(finishes[n]["timestamp"]) for n in t0}
    # ordering
    for nid, spec in graph.nodes.items():
        if nid not in t0:
            continue
        for d in spec.dependencies:
            if d in t1 and t1[d] > t0[nid] + _EPS:
                errors.append(f"dependency {d}->{nid} violated: finish {t1[d]:.6f} > start {t0[nid]:.6f}")
    # exclusivity per resource key
    per_key: Dict[str, List[tuple]] = {}
    for nid in t0:
        for k in graph.nodes[nid].resource_keys:
            per_key.setdefault(k, []).append((t0[nid], t1[nid], nid))
    for k, spans in per_key.items():
        spans.sort()
        for (s_a, f_a, a), (s_b, f_b, b) in zip(spans, spans[1:]):
            if s_b < f_a - _EPS:
                batch = set((starts[a].get("counters") or {}).get("batch_scheduled_nodes") or ())
                if b not in batch:
                    errors.append(f"{a} and {b} overlap on {k}")
    # steps, versions, quantiles, transfers
    taus = _tau_by_name(compiled)
    produced: Dict[str, List[int]] = {}
    emitted: Dict[tuple, int] = {}
    emitted_ranks: Dict[tuple, int] = {}        # a per-rank trace of a data-parallel run counts this rank's share of the rows
    for nid, spec in graph.nodes.items():
        if nid not in finishes:
            continue
        ev = finishes[nid]
        c = ev.get("counters") or {}
        if spec.logical_step is not None and ev.get("step") is not None and int(ev["step"]) != int(spec.logical_step):
            errors.append(f"{nid}: traced step {ev['step']} differs from logical step {spec.logical_step}")
        name = model_name(spec.model)
        if spec.kind is ExecNodeType.OP:
            if name in TRAINABLE_NAMES and spec.role in ("GEN", "INF") and spec.logical_step is not None:
                tau = taus.get(name, 0)
                want = consumer_weight_version(int(spec.logical_step), tau)
                if "weight_version" in c and int(c["weight_version"]) != want:
                    errors.append(f"{nid}: consumed weight version {c['weight_version']}, expected {want}")
                if "shadow" in c and bool(c["shadow"]) != uses_shadow_copies(tau):
                    errors.append(f"{nid}: shadow flag {c['shadow']} inconsistent with tau={tau}")
            if spec.role == "TRAIN" and "produced_weight" in c:
                produced.setdefault(c["produced_weight"]["model"], []).append((t1[nid], int(c["produced_weight"]["version"])))
            en = spec.exec_node
            if en.n_seqs is not None:
                for key, want in (("partial_n_seqs", en.n_seqs), ("partial_n_active", en.n_active),
                                  ("partial_phase_steps", en.phase_steps), ("partial_phase_t_start", en.phase_t_start)):
                    if want is not None and key in c and int(c[key]) != int(want):
                        errors.append(f"{nid}: {key}={c[key]} differs from planned {want}")
                if int(c.get("phase_forced_completions", 0)) != 0:
                    errors.append(f"{nid}: {c['phase_forced_completions']} rows were force-completed at a phase boundary")
            if spec.role == "GEN" and "emitted_rows" in c:
                emitted[(spec.vertex_id, spec.logical_step)] = emitted.get((spec.vertex_id, spec.logical_step), 0) + int(c["emitted_rows"])
                emitted_ranks[(spec.vertex_id, spec.logical_step)] = max(1, int(c.get("data_parallel_ranks", 1)))
        else:
            if "payload_in_bytes" in c and int(c["payload_in_bytes"]) != int(spec.payload_in_bytes):
                errors.append(f"{nid}: transferred {c['payload_in_bytes']} bytes, planned {spec.payload_in_bytes}")
            if "transferred_bytes" in c and "sha256_bytes" in c and int(c["transferred_bytes"]) != int(c["sha256_bytes"]):
                errors.append(f"{nid}: checksum covered {c['sha256_bytes']} of {c['transferred_bytes']} bytes")
    for name, lst in produced.items():
        versions = [v for _, v in sorted(lst)]
        first = versions[0] if versions else 1
        if versions != list(range(first, first + len(versions))):
            errors.append(f"{name}: produced weight versions {versions} are not consecutive")
    if compiled is not None:
        total = compiled.workload.B * compiled.workload.K
        for (vid, step), n in emitted.items():
            want = total // emitted_ranks.get((vid, step), 1)
            if n != want:
                errors.append(f"{vid} step {step}: generation phases emitted {n} rows, expected {want}")
    if attempts["recover"] > attempts["replay"]:
        errors.append("more recover events than replay attempts")
    report = {"ok": not errors, "errors": errors, "warnings": warn, "nodes": len(graph.nodes), "verified_nodes": len(t0),
              "replay_attempts": attempts["replay"], "recoveries": attempts["recover"], "restored_steps": restored_steps, "failed_nodes": sorted(set(failed))}
    if errors and raise_on_error:
        raise RuntimeExecutionError("runtime trace verification failed: " + "; ".join(errors[:8]))
    return report
