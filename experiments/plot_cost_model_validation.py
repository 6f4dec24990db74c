"""Cost-model validation statistics and a predicted-against-measured scatter from calibration reports.

    python experiments/plot_cost_model_validation.py report_a.json report_b.json [--output validation.svg]

Each report is the JSON that ``python -m rpeg_b200.runtime.cost_calibration`` prints (one row per executed node with
its predicted and measured seconds). Per node class (generation / inference / training / transfers) and overall the
script reports the mean absolute percentage error, R^2 of log(predicted) against log(measured), and the share of
nodes predicted within +-25 % - the three figures of the reference's validation across machines
(experiments/plot_cost_model_validation.py:104-108, 782-832) - and draws the log-log scatter with the y = x line.
"""
from __future__ import annotations

import argparse
import json
import math
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from rpeg_b200.utils.visualize import chart_svg  # noqa: E402


def validation_stats(pairs):
    """``pairs`` = [(predicted_s, measured_s)] with positive entries."""
    pairs = [(p, m) for p, m in pairs if p > 0 and m > 0]
    if not pairs:
        return {"n": 0}
    mape = sum(abs(p - m) / m for p, m in pairs) / len(pairs)
    lp, lm = [math.log(p) for p, _ in pairs], [math.log(m) for _, m in pairs]
    mean = sum(lm) / len(lm)
    ss_tot = sum((v - mean) ** 2 for v in lm)
    ss_res = sum((a - b) ** 2 for a, b in zip(lp, lm))
    r2 = 1.0 - ss_res / ss_tot if ss_tot > 0 else (1.0 if ss_res == 0 else float("nan"))
    within = sum(1 for p, m in pairs if abs(p - m) / m <= 0.25) / len(pairs)
    return {"n": len(pairs), "mape": mape, "log_r2": r2, "within_25pct": within}


def load_rows(paths):
    rows = []
    for path in paths:
        text = Path(path).read_text()
        rep = json.loads(text[text.index("{"):])
        for r in rep.get("nodes", ()):
            rows.append((Path(path).stem, r["class"], float(r["predicted_s"]), float(r["measured_s"])))
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("reports", nargs="+")
    ap.add_argument("--output", default=None, help="SVG scatter (log-log) of predicted against measured seconds")
    ap.add_argument("--min-seconds", type=float, default=0.05, help="ignore nodes measured below this (rule rewards, empty transfers)")
    args = ap.parse_args(argv)
    rows = [r for r in load_rows(args.reports) if r[3] >= args.min_seconds]
    classes = sorted({c for _, c, _, _ in rows})
    out = {"reports": [str(p) for p in args.reports], "overall": validation_stats([(p, m) for _, _, p, m in rows]),
           "classes": {c: validation_stats([(p, m) for _, cc, p, m in rows if cc == c]) for c in classes}}
    if args.output:
        chart_svg([(c, [(m, p) for _, cc, p, m in rows if cc == c]) for c in classes], args.output, title="cost model: predicted vs measured",
                  xlabel="measured (s)", ylabel="predicted (s)", log_x=True, log_y=True, lines=False, diagonal=True)
        out["output"] = args.output
    print(json.dumps(out, indent=2))
    return 0 if rows else 1


if __name__ == "__main__":
    sys.exit(main())
