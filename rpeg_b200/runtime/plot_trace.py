"""Render a JSONL runtime trace as an SVG Gantt chart:

    python -m rpeg_b200.runtime.plot_trace --trace traces/run.jsonl [--config run.yaml] --output run.gantt.svg

With ``--config`` the lanes are the GPUs of the run's device space (idle GPUs show as empty lanes);
without it only resources that appear in the trace get a lane. Reference: RPEG/runtime/plot_trace.py.
"""
from __future__ import annotations

import argparse
import sys
from typing import List, Optional

from ..core.types import DeviceSpace
from ..utils.visualize import runtime_trace_to_gantt_svg
from .errors import RuntimeConfigError
from .schema import RuntimeRunConfig
from .trace import read_trace


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="Runtime trace -> SVG Gantt chart")
    ap.add_argument("--trace", required=True)
    ap.add_argument("--config", default=None, help="run file; gives the device space and the title")
    ap.add_argument("--output", required=True)
    args = ap.parse_args(argv)
    try:
        events = read_trace(args.trace)
        space, title = None, "runtime trace"
        if args.config:
            run = RuntimeRunConfig.load(args.config)
            space = DeviceSpace(run.device_space.racks, run.device_space.nodes_per_rack, run.device_space.gpus_per_node)
            title = f"{run.run_id} ({run.algorithm.name})"
        runtime_trace_to_gantt_svg(events, args.output, space, title)
    except (RuntimeConfigError, OSError, ValueError) as exc:
        print(f"runtime error: {exc}", file=sys.stderr)
        return 2
    print(f"wrote {args.output} ({len(events)} events)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
