"""Strong-scaling chart from benchmark result lines: speed-up and efficiency against the number of GPUs.

    python bench.py --gpus 1 > n1.json ; torchrun ... bench.py --gpus 8 > n8.json
    python experiments/plot_strong_scaling.py n1.json n2.json n4.json n8.json --output strong_scaling.svg

Every input file holds JSON objects (one per line, or one JSON list) with ``n_gpus`` and ``value`` (the whole-job rate
``bench.py`` prints; ``--key`` selects another field, ``--series-key`` splits the points into several curves, e.g. by
``impl``). The chart shows the measured rate relative to the smallest GPU count of each series next to the ideal
line; the table printed to stdout gives rate, speed-up and parallel efficiency per point. The reference plots the
PLANNED throughput of a 13B model from 8 to 128 GPUs out of its planner logs (experiments/plot_strong_scaling.py);
``experiments/run_scaling.py`` covers that planned-throughput chart, this script the measured one.
"""
from __future__ import annotations

import argparse
import json
import sys
from collections import defaultdict
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from rpeg_b200.utils.visualize import chart_svg  # noqa: E402


def read_points(files: Sequence[str], key: str = "value", series_key: Optional[str] = None) -> Dict[str, List[Tuple[int, float]]]:
    out: Dict[str, List[Tuple[int, float]]] = defaultdict(list)
    for f in files:
        text = Path(f).read_text().strip()
        if not text:
            continue
        try:
            objs = json.loads(text)
            objs = objs if isinstance(objs, list) else [objs]
        except json.JSONDecodeError:
            objs = []
            for line in text.splitlines():
                line = line.strip()
                if line.startswith("{"):
                    try:
                        objs.append(json.loads(line))
                    except json.JSONDecodeError:
                        continue
        for o in objs:
            if isinstance(o, dict) and o.get(key) is not None and o.get("n_gpus"):
                out[str(o.get(series_key, "measured")) if series_key else "measured"].append((int(o["n_gpus"]), float(o[key])))
    return {k: sorted(v) for k, v in out.items()}


def scaling_table(points: List[Tuple[int, float]], higher_is_better: bool = True) -> List[Dict[str, float]]:
    """Speed-up and efficiency of every point against the series' smallest GPU count."""
    n0, v0 = points[0]
    rows = []
    for n, v in points:
        speedup = (v / v0) if higher_is_better else (v0 / v)
        rows.append({"gpus": n, "value": v, "speedup": speedup, "efficiency": speedup / (n / n0)})
    return rows


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("files", nargs="+")
    ap.add_argument("--key", default="value")
    ap.add_argument("--series-key", default=None)
    ap.add_argument("--lower-is-better", action="store_true", help="the value is a time, not a rate")
    ap.add_argument("--output", default="strong_scaling.svg")
    args = ap.parse_args(argv)
    series = read_points(args.files, args.key, args.series_key)
    if not series:
        print("no points with n_gpus and the requested key", file=sys.stderr)
        return 2
    curves = []
    all_n = sorted({n for pts in series.values() for n, _ in pts})
    for name, pts in sorted(series.items()):
        rows = scaling_table(pts, not args.lower_is_better)
        curves.append((name, [(r["gpus"], r["speedup"]) for r in rows]))
        for r in rows:
            print(f"{name}: {r['gpus']} GPU(s)  {args.key} {r['value']:.4g}  speed-up {r['speedup']:.2f}x  efficiency {100 * r['efficiency']:.0f} %")
    curves.append(("ideal", [(n, n / all_n[0]) for n in all_n]))
    chart_svg(curves, args.output, title="strong scaling (fixed global batch)", xlabel="GPUs", ylabel=f"speed-up over {all_n[0]} GPU(s)",
              log_x=True, log_y=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
