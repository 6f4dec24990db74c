#!/usr/bin/env python
"""``python pipeline.py --hw hw.yaml --config workload.yaml [--time 600]``: analytical plan search."""
import sys

from rpeg_b200.planner.pipeline import main

if __name__ == "__main__":
    sys.exit(main())
