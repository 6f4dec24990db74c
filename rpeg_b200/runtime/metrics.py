"""Everything derived from a runtime trace after (or during) a run: the summary of aggregates, the
Prometheus text export, rule-driven alerts and a static HTML dashboard, all written atomically.

Aggregates (reference: RPEG/runtime/metrics.py:147-952) cover node counts and wall time, transfers
(bytes and seconds by kind and transport), weight publications and layout switches, generation
(tokens, prefill and decode steps, KV page pool, CUDA-graph replays, tokens/s by wall and by node
time), quantile phases, training (latest losses, non-finite losses, gradient norms, optimizer
seconds), device counters (kernel launches, peak memory), weight versions, checkpoints and replay
attempts. Run-to-run comparison of numeric artifact fingerprints follows :27-144 of the same file.
"""
from __future__ import annotations

import html
import json
import math
from collections import defaultdict
from pathlib import Path
from typing import Any, Dict, Iterable, List, Mapping, Optional, Sequence

from .io import atomic_write_text

SUMMARY_SCHEMA = "rpeg.runtime_summary.v1"
ALERT_SCHEMA = "rpeg.runtime_alerts.v1"
FINGERPRINT_FIELDS = ("sum", "sum_abs", "sum_squares", "min", "max")
LOSS_KEYS = ("loss", "policy_loss", "value_loss", "dpo_loss", "kl", "approx_kl", "reward_mean", "grad_norm",
             "actor_grad_norm", "critic_grad_norm", "accuracy")
# counters summed over all finish events -> summary name
SUM_COUNTERS = {
    "generated_tokens": "generation_tokens", "prompt_tokens": "generation_prompt_tokens", "prefill_calls": "generation_prefill_calls",
    "prefill_tokens": "generation_prefill_tokens", "decode_steps": "generation_decode_steps", "graph_replays": "generation_graph_replays",
    "compactions": "generation_compactions", "host_syncs": "generation_host_syncs", "kv_pages_taken": "kv_pool_pages_taken",
    "kv_pages_returned": "kv_pool_pages_returned", "kv_preemptions": "kv_pool_preemptions", "emitted_rows": "generation_emitted_rows",
    "phase_forced_completions": "quantile_forced_completions", "train_tokens": "train_tokens", "train_microbatches": "train_microbatches",
    "optimizer_steps": "optimizer_steps", "kernel_launches": "kernel_launches", "fused_dp_steps": "fused_dp_optimizer_steps",
    "reduce_scatter_bytes": "gradient_reduce_bytes", "fused_pipeline_events": "fused_pipeline_events",
    "transferred_bytes": "transfer_bytes_moved", "peer_copy_launches": "transfer_peer_copy_launches",
    "layout_switches": "layout_switch_count", "layout_switch_bytes": "layout_switch_bytes", "checkpoint_bytes": "checkpoint_bytes",
    "checkpoint_files": "checkpoint_files", "wait_timeouts": "device_wait_timeouts",
}
MAX_COUNTERS = {"peak_memory_bytes": "cuda_peak_memory_bytes", "kv_bytes": "kv_cache_bytes", "live_slots_peak": "generation_live_slots_peak"}


def _finite(x) -> bool:
    return isinstance(x, (int, float)) and not isinstance(x, bool) and math.isfinite(x)


def summarize_trace(events: Sequence[Mapping[str, Any]]) -> Dict[str, Any]:
    s: Dict[str, Any] = {"schema_version": SUMMARY_SCHEMA}
    starts: Dict[str, Mapping[str, Any]] = {}
    by_kind: Dict[str, int] = defaultdict(int)
    by_role: Dict[str, int] = defaultdict(int)
    dur_kind: Dict[str, float] = defaultdict(float)
    dur_role: Dict[str, float] = defaultdict(float)
    dur_model: Dict[str, float] = defaultdict(float)
    xfer_bytes: Dict[str, int] = defaultdict(int)
    xfer_s: Dict[str, float] = defaultdict(float)
    sums: Dict[str, float] = defaultdict(float)
    maxes: Dict[str, float] = {}
    latest: Dict[str, float] = {}
    nonfinite = 0
    produced: Dict[str, int] = {}
    consumed: Dict[str, List[int]] = defaultdict(list)
    shadow_reads = 0
    phases: Dict[int, Dict[str, float]] = defaultdict(lambda: defaultdict(float))
    steps = set()
    errors: List[dict] = []
    started = finished = 0
    run_ids = set()
    t_first = t_last = None
    gen_node_s = train_node_s = 0.0
    replay = recover = ckpt_saves = ckpt_restores = lifecycle = 0
    per_step_wall: Dict[int, List[float]] = defaultdict(lambda: [math.inf, -math.inf])
    for e in events:
        run_ids.add(e.get("run_id"))
        ts = e.get("timestamp")
        if _finite(ts):
            t_first = ts if t_first is None else min(t_first, ts)
            t_last = ts if t_last is None else max(t_last, ts)
        ev, nid = e.get("event"), e.get("node_id")
        c = e.get("counters") or {}
        if ev == "replay":
            replay += 1
            continue
        if ev == "recover":
            recover += 1
            continue
        if nid == "runtime.checkpoint.save" and ev == "finish":
            ckpt_saves += 1
            for k in ("checkpoint_bytes", "checkpoint_files"):
                if _finite(c.get(k)):
                    sums[SUM_COUNTERS[k]] += c[k]
            continue
        if nid == "runtime.checkpoint.restore" and ev == "finish":
            ckpt_restores += 1
            continue
        if str(nid).startswith("runtime."):      # lifecycle nodes (worker start-up, initial publication) are not graph nodes
            lifecycle += 1 if ev == "finish" else 0
            continue
        if ev == "start":
            started += 1
            starts[nid] = e
            continue
        if ev != "finish":
            continue
        if e.get("status") != "ok":
            errors.append({"node_id": nid, "message": e.get("message"), "step": e.get("step")})
            continue
        finished += 1
        st = starts.get(nid) or {}
        info = {**(st.get("counters") or {}), **c}
        kind, role, model = str(info.get("kind", "op")).lower(), info.get("role"), info.get("model")
        dur = float(c.get("duration_s", (ts - st["timestamp"]) if st and _finite(ts) else 0.0) or 0.0)
        by_kind[kind] += 1
        dur_kind[kind] += dur
        step = e.get("step")
        if step is not None:
            steps.add(int(step))
            w = per_step_wall[int(step)]
            if st and _finite(st.get("timestamp")):
                w[0] = min(w[0], st["timestamp"])
            if _finite(ts):
                w[1] = max(w[1], ts)
        if kind == "op":
            if role:
                by_role[role] += 1
                dur_role[role] += dur
            if model:
                dur_model[model] += dur
            if role == "GEN":
                gen_node_s += dur
            if role == "TRAIN":
                train_node_s += dur
            if "weight_version" in c and model:
                consumed[model].append(int(c["weight_version"]))
                shadow_reads += 1 if c.get("shadow") else 0
            pw = c.get("produced_weight")
            if pw:
                produced[pw["model"]] = max(produced.get(pw["model"], 0), int(pw["version"]))
            if "artifact_part" in c:
                ph = phases[int(c["artifact_part"])]
                ph["nodes"] += 1
                ph["seconds"] += dur
                ph["planned_rows"] += float(c.get("partial_n_seqs", 0))
                ph["emitted_rows"] += float(c.get("emitted_rows", 0))
            for k in LOSS_KEYS:
                if k in c:
                    if _finite(c[k]):
                        latest[k] = float(c[k])
                    else:
                        nonfinite += 1
        else:
            transport = str(c.get("transport", "metadata"))
            label = "weight" if str(info.get("label") or "").startswith("W_") else "activation"
            nbytes = int(c.get("transferred_bytes", c.get("payload_in_bytes", 0)) or 0)
            for key in (kind, label, f"transport_{transport}"):
                xfer_bytes[key] += nbytes
                xfer_s[key] += dur
        for k, name in SUM_COUNTERS.items():
            if _finite(c.get(k)):
                sums[name] += c[k]
        for k, name in MAX_COUNTERS.items():
            if _finite(c.get(k)):
                maxes[name] = max(maxes.get(name, 0.0), float(c[k]))
    wall = (t_last - t_first) if t_first is not None else 0.0
    s.update(run_id=next(iter(run_ids)) if len(run_ids) == 1 else sorted(map(str, run_ids)), event_count=len(events),
             nodes_started=started, nodes_finished=finished, nodes_failed=len(errors), nodes_incomplete=max(0, started - finished - len(errors)),
             wall_time_s=wall, logical_steps=len(steps), first_step=min(steps) if steps else None, last_step=max(steps) if steps else None,
             replay_attempts=replay, recoveries=recover, checkpoint_saves=ckpt_saves, checkpoint_restores=ckpt_restores,
             errors=errors[:20], nonfinite_losses=nonfinite, lifecycle_nodes=lifecycle)
    for k, v in by_kind.items():
        s[f"nodes_{k}"] = v
        s[f"node_seconds_{k}"] = dur_kind[k]
    for k, v in by_role.items():
        s[f"operators_{k.lower()}"] = v
        s[f"operator_seconds_{k.lower()}"] = dur_role[k]
    for k, v in dur_model.items():
        s[f"operator_seconds_model_{k}"] = v
    for k, v in xfer_bytes.items():
        s[f"transfer_bytes_{k}"] = v
        s[f"transfer_seconds_{k}"] = xfer_s[k]
        s[f"transfer_gbps_{k}"] = (v / xfer_s[k] / 1e9) if xfer_s[k] > 0 else 0.0
    s.update({k: (int(v) if float(v).is_integer() else v) for k, v in sums.items()})
    s.update(maxes)
    s.update({f"latest_{k}": v for k, v in latest.items()})
    tok = float(sums.get("generation_tokens", 0.0))
    s["generation_tokens_per_s_wall"] = tok / wall if wall > 0 else 0.0
    s["generation_tokens_per_s_node"] = tok / gen_node_s if gen_node_s > 0 else 0.0
    s["train_tokens_per_s_node"] = float(sums.get("train_tokens", 0.0)) / train_node_s if train_node_s > 0 else 0.0
    s["kv_pool_pages_outstanding"] = int(sums.get("kv_pool_pages_taken", 0) - sums.get("kv_pool_pages_returned", 0))
    busy = sum(dur_kind.values())
    s["node_seconds_total"] = busy
    s["overlap_factor"] = busy / wall if wall > 0 else 0.0
    s["weight_versions_produced"] = dict(produced)
    s["weight_versions_consumed_max"] = {m: max(v) for m, v in consumed.items()}
    s["weight_version_lag_max"] = {m: max(0, produced.get(m, 0) - min(v)) for m, v in consumed.items()}
    s["weight_shadow_reads"] = shadow_reads
    s["quantile_phases"] = {str(k): dict(v) for k, v in sorted(phases.items())}
    s["step_wall_s"] = {str(k): (v[1] - v[0]) for k, v in sorted(per_step_wall.items()) if v[1] >= v[0]}
    if s["step_wall_s"]:
        vals = list(s["step_wall_s"].values())
        s["step_wall_s_mean"], s["step_wall_s_max"] = sum(vals) / len(vals), max(vals)
    return s


def compare_artifact_numeric_fingerprints(a: Mapping[str, Mapping[str, Any]], b: Mapping[str, Mapping[str, Any]], *,
                                          atol: float = 1e-6, rtol: float = 1e-5) -> Dict[str, Any]:
    """Compare two runs' artifact fingerprints (moments per named tensor). Integer and boolean
    tensors must match exactly, floating ones within ``atol + rtol*|b|``; counts always exactly."""
    mismatches: List[dict] = []
    for name in sorted(set(a) | set(b)):
        fa, fb = a.get(name), b.get(name)
        if fa is None or fb is None:
            mismatches.append({"artifact": name, "field": "presence", "a": fa is not None, "b": fb is not None})
            continue
        for f in ("count", "dtype", "shape"):
            if f in fa or f in fb:
                if fa.get(f) != fb.get(f):
                    mismatches.append({"artifact": name, "field": f, "a": fa.get(f), "b": fb.get(f)})
        exact = str(fa.get("dtype", "")).startswith(("int", "uint", "bool", "torch.int", "torch.uint", "torch.bool"))
        for f in FINGERPRINT_FIELDS:
            if f not in fa and f not in fb:
                continue
            x, y = fa.get(f), fb.get(f)
            if x is None or y is None:
                ok = x == y
            elif exact:
                ok = x == y
            elif not (_finite(x) and _finite(y)):
                ok = (isinstance(x, float) and isinstance(y, float) and math.isnan(x) and math.isnan(y)) or x == y
            else:
                ok = abs(x - y) <= atol + rtol * abs(y)
            if not ok:
                mismatches.append({"artifact": name, "field": f, "a": x, "b": y})
    return {"ok": not mismatches, "compared": len(set(a) & set(b)), "mismatches": mismatches}


def tensor_fingerprint(t) -> Dict[str, Any]:
    """Moments of a tensor for run-to-run comparison (computed in float64 on the tensor's device)."""
    import torch
    x = t.detach()
    out: Dict[str, Any] = {"count": int(x.numel()), "dtype": str(x.dtype).replace("torch.", ""), "shape": list(x.shape)}
    if x.numel() == 0:
        return out
    if x.dtype == torch.bool or not x.dtype.is_floating_point:
        xi = x.to(torch.int64)
        out.update(sum=int(xi.sum()), sum_abs=int(xi.abs().sum()), sum_squares=int((xi * xi).sum()), min=int(xi.min()), max=int(xi.max()))
    else:
        xd = x.to(torch.float64)
        out.update(sum=float(xd.sum()), sum_abs=float(xd.abs().sum()), sum_squares=float((xd * xd).sum()), min=float(xd.min()),
                   max=float(xd.max()))
    return out


# ------------------------------------------------------------------------------ Prometheus text
def _metric_name(key: str) -> str:
    out = "".join(ch if ch.isalnum() else "_" for ch in key.lower())
    return "rpeg_runtime_" + out.strip("_")


def prometheus_text(summary: Mapping[str, Any], labels: Optional[Mapping[str, str]] = None) -> str:
    """Prometheus exposition text: every scalar aggregate becomes a gauge ``rpeg_runtime_<name>``;
    dictionaries of scalars become one gauge with a ``key`` label."""
    base = {"run_id": str(summary.get("run_id", "")), **dict(labels or {})}

    def fmt_labels(extra: Mapping[str, str] = {}) -> str:
        items = {**base, **extra}
        return "{" + ",".join(f'{k}="{str(v).replace(chr(92), chr(92) * 2).replace(chr(34), chr(92) + chr(34))}"'
                              for k, v in items.items()) + "}"

    lines: List[str] = []
    for key in sorted(summary):
        val = summary[key]
        name = _metric_name(key)
        if isinstance(val, bool):
            val = int(val)
        if _finite(val):
            lines += [f"# TYPE {name} gauge", f"{name}{fmt_labels()} {val}"]
        elif isinstance(val, Mapping) and val and all(_finite(v) for v in val.values()):
            lines.append(f"# TYPE {name} gauge")
            lines += [f"{name}{fmt_labels({'key': str(k)})} {v}" for k, v in val.items()]
        elif isinstance(val, Mapping) and val and all(isinstance(v, Mapping) for v in val.values()):
            for sub in sorted({f for v in val.values() for f in v}):
                lines.append(f"# TYPE {name}_{sub} gauge")
                lines += [f"{name}_{sub}{fmt_labels({'key': str(k)})} {v[sub]}" for k, v in val.items() if _finite(v.get(sub))]
    return "\n".join(lines) + "\n"


# ------------------------------------------------------------------------------ alerts
DEFAULT_ALERT_RULES = {"max_nodes_failed": 0, "max_nodes_incomplete": 0, "max_nonfinite_losses": 0, "max_device_wait_timeouts": 0,
                       "max_replay_attempts": 0, "max_kv_pool_pages_outstanding": 0, "max_quantile_forced_completions": 0}


def evaluate_alerts(summary: Mapping[str, Any], rules: Optional[Mapping[str, Any]] = None,
                    verification: Optional[Mapping[str, Any]] = None) -> Dict[str, Any]:
    """Rules are ``min_<aggregate>``, ``max_<aggregate>`` or ``require_<aggregate>``; a rule's value
    is either the bound or ``{value: ..., severity: warning|critical}``. Defaults flag failed or
    incomplete nodes, non-finite losses, device wait timeouts, replays, leaked KV pages and forced
    phase completions. A failed trace verification is always critical."""
    merged = {**DEFAULT_ALERT_RULES, **dict(rules or {})}
    alerts: List[dict] = []
    for rule, spec in merged.items():
        bound, severity = (spec.get("value"), spec.get("severity", "critical")) if isinstance(spec, Mapping) else (spec, "critical")
        if bound is None:
            continue
        if rule.startswith("max_"):
            key, actual = rule[4:], summary.get(rule[4:], 0)
            bad = _finite(actual) and actual > bound
        elif rule.startswith("min_"):
            key, actual = rule[4:], summary.get(rule[4:])
            bad = actual is None or (_finite(actual) and actual < bound)
        elif rule.startswith("require_"):
            key, actual = rule[8:], summary.get(rule[8:])
            bad = bool(bound) and not actual
        else:
            alerts.append({"rule": rule, "severity": "warning", "message": f"unknown alert rule {rule!r} ignored"})
            continue
        if bad:
            alerts.append({"rule": rule, "aggregate": key, "bound": bound, "actual": actual, "severity": severity,
                           "message": f"{key}={actual} violates {rule}={bound}"})
    if verification is not None and not verification.get("ok", True):
        alerts.append({"rule": "trace_verification", "severity": "critical", "actual": len(verification.get("errors", ())),
                       "message": "; ".join(list(verification.get("errors", ()))[:3])})
    worst = "critical" if any(a["severity"] == "critical" for a in alerts) else ("warning" if alerts else "ok")
    return {"schema_version": ALERT_SCHEMA, "run_id": summary.get("run_id"), "status": worst, "alert_count": len(alerts),
            "alerts": alerts, "rules": merged}


# ------------------------------------------------------------------------------ dashboard
def dashboard_html(summary: Mapping[str, Any], alerts: Optional[Mapping[str, Any]] = None, gantt_svg: Optional[str] = None) -> str:
    esc = html.escape
    status = (alerts or {}).get("status", "ok")
    colour = {"ok": "#2e7d32", "warning": "#f9a825", "critical": "#c62828"}.get(status, "#555")
    head = ["nodes_finished", "nodes_failed", "wall_time_s", "logical_steps", "generation_tokens", "generation_tokens_per_s_wall",
            "train_tokens", "kernel_launches", "cuda_peak_memory_bytes", "replay_attempts", "latest_loss", "latest_grad_norm"]
    cards = "".join(f'<div class="card"><div class="k">{esc(k)}</div><div class="v">{esc(_fmt(summary[k]))}</div></div>'
                    for k in head if k in summary)
    rows = "".join(f"<tr><td>{esc(k)}</td><td>{esc(_fmt(v))}</td></tr>" for k, v in sorted(summary.items())
                   if not isinstance(v, (Mapping, list)))
    nested = "".join(f"<h3>{esc(k)}</h3><pre>{esc(json.dumps(v, indent=1, default=str))}</pre>" for k, v in sorted(summary.items())
                     if isinstance(v, (Mapping, list)) and v)
    alert_rows = "".join(f'<tr><td>{esc(a["severity"])}</td><td>{esc(a["rule"])}</td><td>{esc(str(a.get("message", "")))}</td></tr>'
                         for a in (alerts or {}).get("alerts", ()))
    return f"""<!doctype html><html><head><meta charset="utf-8"><title>RPEG run {esc(str(summary.get('run_id', '')))}</title>
<style>body{{font-family:sans-serif;margin:24px}} .card{{display:inline-block;border:1px solid #ccc;border-radius:6px;padding:8px 14px;margin:4px}}
.k{{font-size:11px;color:#666}} .v{{font-size:18px}} table{{border-collapse:collapse}} td{{border-bottom:1px solid #eee;padding:2px 10px;font-family:monospace;font-size:12px}}
.status{{color:white;background:{colour};padding:3px 10px;border-radius:4px}}</style></head><body>
<h1>RPEG runtime: {esc(str(summary.get('run_id', '')))} <span class="status">{esc(status)}</span></h1>
<div>{cards}</div>
<h2>Alerts</h2><table>{alert_rows or '<tr><td>none</td></tr>'}</table>
{('<h2>Timeline</h2>' + gantt_svg) if gantt_svg else ''}
<h2>Aggregates</h2><table>{rows}</table>{nested}
</body></html>"""


def _fmt(v) -> str:
    if isinstance(v, float):
        return f"{v:.6g}"
    return str(v)


# ------------------------------------------------------------------------------ writers
def write_runtime_summary(events: Sequence[Mapping[str, Any]], *, summary_path=None, metrics_path=None, alert_path=None,
                          dashboard_path=None, alert_rules: Optional[Mapping[str, Any]] = None,
                          verification: Optional[Mapping[str, Any]] = None, extra: Optional[Mapping[str, Any]] = None,
                          gantt_svg: Optional[str] = None) -> Dict[str, Any]:
    summary = summarize_trace(events)
    if extra:
        summary.update(extra)
    alerts = evaluate_alerts(summary, alert_rules, verification)
    if summary_path:
        atomic_write_text(summary_path, json.dumps(summary, indent=2, default=str))
    if metrics_path:
        atomic_write_text(metrics_path, prometheus_text(summary))
    if alert_path:
        atomic_write_text(alert_path, json.dumps(alerts, indent=2, default=str))
    if dashboard_path:
        atomic_write_text(dashboard_path, dashboard_html(summary, alerts, gantt_svg))
    return {"summary": summary, "alerts": alerts}


def write_runtime_summary_for_run(run_config, events: Sequence[Mapping[str, Any]], verification=None, extra=None) -> Dict[str, Any]:
    m = run_config.monitoring
    res = lambda p: None if not p else run_config.resolve(p)
    return write_runtime_summary(events, summary_path=res(m.summary_path), metrics_path=res(m.metrics_path),
                                 alert_path=res(m.alert_path), dashboard_path=res(m.dashboard_path), alert_rules=m.alert_rules,
                                 verification=verification, extra=extra)
