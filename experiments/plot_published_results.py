"""Tables and charts of the published end-to-end PPO measurements.

    python experiments/plot_published_results.py --results final_results.tar.bz2 [--out-dir figures/published]

The measurements ship as an archive of ``athena_results/<GPUs>-<model size in B>/metrics_report.json`` files (a
directory with the same layout works too). Each report holds, per schedule (``pardistrlm`` = the plan found by the
optimizer, ``native`` = the baseline system's own plan), ``runtime.benchmark_wall_time_s``, ``runtime.tokens_per_s``
and ``runtime.hardware_utilization.avg_utilization_pct``. This tool prints one row per (model, GPU count) with both
schedules and the speed-up, and writes three SVG charts (iteration time, throughput, utilisation against the GPU
count, one line per model and schedule). Reference: paper/plots.py:21-36 (metric paths, labels), :78-277 (the figure).
"""
from __future__ import annotations

import argparse
import json
import sys
import tarfile
from pathlib import Path
from typing import Dict, Iterator, List, Optional, Tuple

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

SCHEDULES = {"pardistrlm": "RPEG plan", "native": "baseline plan"}
METRICS = {
    "iteration_s": ("benchmark_wall_time_s",),
    "tokens_per_s": ("tokens_per_s",),
    "utilization_pct": ("hardware_utilization", "avg_utilization_pct"),
}


def _reports(source: Path) -> Iterator[Tuple[str, dict]]:
    """(``"<GPUs>-<model>"``, report) for every ``metrics_report.json`` in an archive or a directory."""
    if source.is_dir():
        for p in sorted(source.rglob("metrics_report.json")):
            yield p.parent.name, json.loads(p.read_text())
        return
    with tarfile.open(source) as tar:
        for member in sorted(tar.getmembers(), key=lambda m: m.name):
            if member.isfile() and member.name.endswith("metrics_report.json"):
                yield Path(member.name).parent.name, json.load(tar.extractfile(member))


def _dig(d: Optional[dict], path: Tuple[str, ...]) -> Optional[float]:
    for key in path:
        if not isinstance(d, dict) or d.get(key) is None:
            return None
        d = d[key]
    return float(d)


def load(source: Path) -> List[dict]:
    """One row per run directory: GPUs, model size, and every metric of both schedules (``None`` where absent)."""
    rows = []
    for name, rep in _reports(source):
        try:
            gpus, model = (int(x) for x in name.split("-", 1))
        except ValueError:
            continue
        row = {"gpus": gpus, "model_b": model}
        for sched in SCHEDULES:
            rt = ((rep.get("schedules") or {}).get(sched) or {}).get("runtime")
            for metric, path in METRICS.items():
                row[f"{sched}.{metric}"] = _dig(rt, path)
        a, b = row["pardistrlm.iteration_s"], row["native.iteration_s"]
        row["speedup"] = (b / a) if (a and b) else None
        rows.append(row)
    rows.sort(key=lambda r: (r["model_b"], r["gpus"]))
    return rows


def table(rows: List[dict]) -> str:
    fmt = lambda v, spec: "-" if v is None else format(v, spec)  # noqa: E731
    out = [f"{'model':>6} {'GPUs':>5} | {'RPEG s':>9} {'tok/s':>9} {'util %':>7} | {'base s':>9} {'tok/s':>9} {'util %':>7} | {'speed-up':>8}"]
    for r in rows:
        out.append(f"{r['model_b']:>5}B {r['gpus']:>5} | {fmt(r['pardistrlm.iteration_s'], '9.2f')} {fmt(r['pardistrlm.tokens_per_s'], '9.2f')} "
                   f"{fmt(r['pardistrlm.utilization_pct'], '7.1f')} | {fmt(r['native.iteration_s'], '9.2f')} "
                   f"{fmt(r['native.tokens_per_s'], '9.2f')} {fmt(r['native.utilization_pct'], '7.1f')} | {fmt(r['speedup'], '8.2f')}")
    return "\n".join(out)


def charts(rows: List[dict], out_dir: Path) -> List[Path]:
    from rpeg_b200.utils.visualize import chart_svg
    out_dir.mkdir(parents=True, exist_ok=True)
    written = []
    for metric, label in (("iteration_s", "PPO iteration (s)"), ("tokens_per_s", "tokens / s"), ("utilization_pct", "GPU utilisation (%)")):
        series: Dict[str, List[Tuple[float, float]]] = {}
        for r in rows:
            for sched, name in SCHEDULES.items():
                v = r[f"{sched}.{metric}"]
                if v is not None:
                    series.setdefault(f"{r['model_b']}B, {name}", []).append((float(r["gpus"]), v))
        if not series:
            continue
        path = out_dir / f"published_{metric}.svg"
        chart_svg(sorted(series.items()), str(path), title=f"published measurements: {label}", xlabel="GPUs", ylabel=label, log_x=True)
        written.append(path)
    return written


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--results", required=True, help="final_results.tar.bz2, or a directory of <GPUs>-<model>/metrics_report.json")
    ap.add_argument("--out-dir", default=None, help="write the SVG charts here")
    ap.add_argument("--json", action="store_true", help="print the rows as JSON instead of a table")
    args = ap.parse_args(argv)
    rows = load(Path(args.results))
    if not rows:
        print(f"no metrics_report.json under {args.results}", file=sys.stderr)
        return 1
    print(json.dumps(rows, indent=1) if args.json else table(rows))
    if args.out_dir:
        for p in charts(rows, Path(args.out_dir)):
            print(f"wrote {p}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
