"""Rank process used by the control-plane tests and by ``runtime.dist_validate``: it joins the
job's process group, reports heartbeats and runs a small loop of collective "steps" on the CPU
(gloo) or on its GPU (nccl).

    python -m rpeg_b200.runtime.worker_entry --steps 3 [--backend gloo|nccl] [--step-sleep 0.05]

Host-side failure injection (never on the device), through the environment:
  RPEG_TEST_FAIL_RANK=<r>            the rank that fails (default: all ranks, if an operation is named)
  RPEG_TEST_FAIL_OPERATION=init|step|never_ready|exit
      init         raise before the process group is joined
      step         raise between steps, at step RPEG_TEST_FAIL_STEP (default 1), with no collective in flight
      never_ready  sleep without ever reporting ``ready``
      exit         leave with exit code 3 between steps without reporting
A rank that sees a peer's ``error`` heartbeat before its next collective stops cleanly instead of
entering a collective that can never complete. Reference: RPEG/runtime/worker_entry.py:90 and the
injection hook RPEG/runtime/semantic_worker.py:311-326.
"""
from __future__ import annotations

import argparse
import datetime
import os
import sys
import time
from typing import List, Optional

from .control import HeartbeatStore


def peer_failed(store: HeartbeatStore, group: str, world: int, me: int) -> Optional[int]:
    for r in range(world):
        if r == me:
            continue
        hb = store.read(group, r)
        if hb is not None and hb.state == "error":
            return r
    return None


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--backend", default="gloo", choices=("gloo", "nccl"))
    ap.add_argument("--step-sleep", type=float, default=0.0)
    ap.add_argument("--collective-timeout", type=float, default=10.0)
    args = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    group = os.environ.get("RPEG_GROUP_ID", "group")
    store = HeartbeatStore(os.environ.get("RPEG_HEARTBEAT_DIR", "heartbeats"))
    fail_op = os.environ.get("RPEG_TEST_FAIL_OPERATION")
    fail_rank = os.environ.get("RPEG_TEST_FAIL_RANK")
    fail_step = int(os.environ.get("RPEG_TEST_FAIL_STEP", "1"))
    mine = fail_op is not None and (fail_rank is None or int(fail_rank) == rank)
    store.write(group, rank, "starting")
    try:
        if mine and fail_op == "never_ready":
            time.sleep(3600)
        if mine and fail_op == "init":
            raise RuntimeError("injected failure during initialisation")
        import torch
        import torch.distributed as dist
        if args.backend == "nccl":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group(args.backend, timeout=datetime.timedelta(seconds=args.collective_timeout))
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if args.backend == "nccl" else torch.device("cpu")
        store.write(group, rank, "ready")
        total = 0.0
        for step in range(1, args.steps + 1):
            # between steps nothing is in flight: this is where a rank may fail or leave
            if mine and fail_op == "step" and step == fail_step:
                raise RuntimeError(f"injected failure before step {step}")
            if mine and fail_op == "exit" and step == fail_step:
                os._exit(3)
            bad = peer_failed(store, group, world, rank)
            if bad is not None:
                store.write(group, rank, "stopped", message=f"peer rank {bad} failed before step {step}", step=step)
                return 4
            store.write(group, rank, "running", step=step)
            x = torch.full((4,), float(rank + step), device=dev)
            dist.all_reduce(x)
            total += float(x[0])
            if args.step_sleep:
                time.sleep(args.step_sleep)
        expect = sum(sum(r + s for r in range(world)) for s in range(1, args.steps + 1))
        if abs(total - expect) > 1e-6:
            raise RuntimeError(f"all-reduce check failed: {total} != {expect}")
        store.write(group, rank, "finished", message=f"sum={total}")
        dist.destroy_process_group()
        return 0
    except Exception as exc:       # report, then leave with a non-zero code so the launcher aborts the group
        store.write(group, rank, "error", message=f"{type(exc).__name__}: {exc}")
        return 1


if __name__ == "__main__":
    sys.exit(main())
