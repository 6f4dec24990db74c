"""Per-operator time of the planner's input plan against its optimised plan, as grouped bars.

    python -m rpeg_b200.runtime.job_plan --config job.yaml --out-dir /tmp/job
    python experiments/plot_operator_breakdown.py /tmp/job/metrics/analytical_comparison.json --output breakdown.svg
    python experiments/plot_operator_breakdown.py a.json b.json --by kind --output kinds.svg

Input: one or more ``analytical_comparison.json`` files written by ``runtime.job_plan`` (they carry the scheduled
seconds of the baseline and the optimised plan per template vertex and per operator class). With one file the groups
are the operators (generation, the inference vertices, the training vertices) and the bars "input" and "optimized";
with several files every file becomes one group per plan. ``--trace run.jsonl`` adds the MEASURED seconds of a runtime
trace of the optimised plan as a third bar. The reference draws the same comparison (greedy / concurrent heuristic /
optimised, per operator) from a results file with matplotlib (experiments/plot_operator_breakdown.py).
"""
from __future__ import annotations

import argparse
import json
import sys
from collections import defaultdict
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from rpeg_b200.utils.visualize import bars_svg  # noqa: E402

ORDER = ("g_pi", "g_ac", "i_ref", "i_R", "i_V", "i_ac", "i_pi", "t_pi", "t_ac", "t_V")
LABEL = {"g_pi": "actor\ngen.", "g_ac": "shared\ngen.", "i_ref": "ref.\ninf.", "i_R": "reward\ninf.", "i_V": "critic\ninf.",
         "i_ac": "shared\ninf.", "i_pi": "actor\ninf.", "t_pi": "actor\ntrain", "t_ac": "shared\ntrain", "t_V": "critic\ntrain",
         "GEN": "generation", "INF": "inference", "TRAIN": "training", "comm": "transfers", "reshard": "layout\nswitches"}


def measured_seconds(trace_path: str, by: str) -> Dict[str, float]:
    """Sum of the finish events' durations per vertex (or per class) of a runtime trace."""
    out: Dict[str, float] = defaultdict(float)
    for line in Path(trace_path).read_text().splitlines():
        if not line.strip():
            continue
        e = json.loads(line)
        if e.get("event") != "finish":
            continue
        vid = str(e.get("node_id", "")).split("@")[0]
        dur = float((e.get("counters") or {}).get("duration_s", e.get("duration_s", 0.0)) or 0.0)
        if by == "vertex":
            out[vid] += dur
        else:
            kind = {"g": "GEN", "i": "INF", "t": "TRAIN"}.get(vid[:1]) if "_" in vid[:3] else None
            out[kind or ("reshard" if "reshard" in vid else "comm")] += dur
    return dict(out)


def breakdown_groups(files: Sequence[str], by: str = "vertex", trace: Optional[str] = None) -> List[Tuple[str, List[Tuple[str, float]]]]:
    key = "seconds_by_vertex" if by == "vertex" else "seconds_by_kind"
    reports = [(Path(f), json.loads(Path(f).read_text())) for f in files]
    for path, rep in reports:
        if key not in rep.get("output", {}):
            raise SystemExit(f"{path}: no {key} (written by runtime.job_plan of this version)")
    groups: List[Tuple[str, List[Tuple[str, float]]]] = []
    if len(reports) == 1:
        _, rep = reports[0]
        meas = measured_seconds(trace, by) if trace else {}
        ops = [o for o in (ORDER if by == "vertex" else ("GEN", "INF", "TRAIN", "comm", "reshard")) if o in rep["output"][key] or o in rep["input"].get(key, {})]
        ops += sorted(set(rep["output"][key]) - set(ops))
        for op in ops:
            bars = [("input plan", float(rep["input"].get(key, {}).get(op, 0.0))), ("optimized plan", float(rep["output"][key].get(op, 0.0)))]
            if trace:
                bars.append(("measured", float(meas.get(op, 0.0))))
            groups.append((LABEL.get(op, op), bars))
        return groups
    for path, rep in reports:
        name = str(rep.get("run_id") or path.parent.parent.name)
        for plan in ("input", "output"):
            groups.append((f"{name}\n{plan}", [(LABEL.get(k, k).replace("\n", " "), float(v)) for k, v in sorted(rep[plan].get(key, {}).items())]))
    return groups


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("files", nargs="+")
    ap.add_argument("--by", choices=("vertex", "kind"), default="vertex")
    ap.add_argument("--trace", default=None, help="runtime trace of the optimised plan (one input file only)")
    ap.add_argument("--output", default="operator_breakdown.svg")
    args = ap.parse_args(argv)
    groups = breakdown_groups(args.files, args.by, args.trace)
    bars_svg(groups, args.output, title="scheduled seconds per operator (all logical steps)", ylabel="seconds")
    for label, bars in groups:
        print(label.replace("\n", " ") + ": " + ", ".join(f"{n} {v:.3f} s" for n, v in bars))
    return 0


if __name__ == "__main__":
    sys.exit(main())
