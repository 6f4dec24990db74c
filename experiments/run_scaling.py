"""Run the plan search over a set of scaling configs and plot throughput against the number of GPUs.

    python experiments/gen_scaling_configs.py --out /tmp/scaling
    python experiments/run_scaling.py /tmp/scaling --match actor/ --time 20 --csv scaling.csv --plot scaling.svg

For every config (a YAML of ``gen_scaling_configs.py``) the planner is run with ``--time`` seconds of search; the
CSV gets one row per config with the predicted tokens/s, makespan and utilisation of the greedy baseline, the
concurrent heuristic and the optimised plan; the chart shows tokens/s of the three against the GPU count. This is
the data the reference extracts from its run logs (experiments/plot_scaling.py:92-168) - here the search is called
as a function, so nothing is parsed.
"""
from __future__ import annotations

import argparse
import contextlib
import csv
import io
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import yaml  # noqa: E402

from rpeg_b200.planner.pipeline import make_yaml_loader, run_pipeline  # noqa: E402
from rpeg_b200.utils.visualize import chart_svg  # noqa: E402


def run_one(path: Path, time_s: float) -> dict:
    cfg = yaml.load(path.read_text(), Loader=make_yaml_loader())
    hw = cfg["hardware"]
    gpus = int(hw["racks"]) * int(hw["nodes_per_rack"]) * int(hw["gpus_per_node"])
    with contextlib.redirect_stdout(io.StringIO()):
        res = run_pipeline(cfg, time_budget_s=time_s, make_plots=False)
    row = {"config": path.name, "gpus": gpus, "search_wall_s": round(res["wall_s"], 2)}
    for key, r in zip(("greedy", "heuristic", "optimized"), res["rows"]):
        if r:
            row.update({f"{key}_tokens_per_s": r["tokens_per_s"], f"{key}_makespan_s": r["makespan_s"], f"{key}_utilization": r.get("utilization")})
    return row


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("configs_dir")
    ap.add_argument("--match", default="", help="substring the path of a config below configs_dir must contain")
    ap.add_argument("--time", type=float, default=20.0, help="search seconds per config")
    ap.add_argument("--limit", type=int, default=0, help="at most this many configs (0 = all)")
    ap.add_argument("--csv", default="scaling.csv")
    ap.add_argument("--plot", default=None)
    args = ap.parse_args(argv)
    paths = sorted(p for p in Path(args.configs_dir).rglob("*.yaml") if args.match in str(p.relative_to(args.configs_dir)))
    if args.limit:
        paths = paths[: args.limit]
    rows = []
    for p in paths:
        try:
            rows.append(run_one(p, args.time))
            print(f"{p.name}: {rows[-1].get('optimized_tokens_per_s', float('nan')):.4g} tok/s on {rows[-1]['gpus']} GPUs", file=sys.stderr)
        except Exception as exc:                       # an infeasible config must not end the sweep
            print(f"{p.name}: skipped ({exc})", file=sys.stderr)
    if not rows:
        print("no config ran", file=sys.stderr)
        return 1
    fields = sorted({k for r in rows for k in r}, key=lambda k: (k not in ("config", "gpus"), k))
    with open(args.csv, "w", newline="") as fh:
        w = csv.DictWriter(fh, fieldnames=fields)
        w.writeheader()
        w.writerows(rows)
    if args.plot:
        series = []
        for key in ("greedy", "heuristic", "optimized"):
            best = {}
            for r in rows:                                 # several configs may share a GPU count: keep the best of each
                v = r.get(f"{key}_tokens_per_s")
                if v:
                    best[r["gpus"]] = max(best.get(r["gpus"], 0.0), float(v))
            if best:
                series.append((key, sorted(best.items())))
        chart_svg(series, args.plot, title=f"predicted throughput ({args.match or 'all configs'})", xlabel="GPUs", ylabel="tokens / s",
                  log_x=True, log_y=True)
    print(f"{len(rows)} config(s) -> {args.csv}" + (f", {args.plot}" if args.plot else ""))
    return 0


if __name__ == "__main__":
    sys.exit(main())
