"""One task of a Slurm step that was started by ``SlurmWorkerGroupLauncher``: look this task up in the step's manifest and
become the rank process it describes.

    srun ... python -m rpeg_b200.runtime.pool_entry --manifest <dir>/launch_manifest.json

``srun`` starts the same command line in every task; what a task is to do is in the manifest
(``rpeg.worker_pool.v1``): ``hosts[<short hostname>][<SLURM_LOCALID>]`` names the task, ``tasks[<id>]`` holds either
``{"idle": true}`` (a filler slot on a host with fewer ranks than the widest one: it waits for the stop file or SIGTERM)
or the rank's environment (``RANK``, ``WORLD_SIZE``, rendezvous, heartbeat directory, group id), its module, arguments
and log file. The module runs in this process, so the step's exit code is the rank's.
Reference: RPEG/runtime/semantic_pool_entry.py:47-88 (the shared-step dispatcher).
"""
from __future__ import annotations

import argparse
import json
import os
import runpy
import signal
import sys
import time
from pathlib import Path
from typing import List, Optional

SCHEMA = "rpeg.worker_pool.v1"


def short_hostname() -> str:
    return (os.environ.get("RPEG_POOL_HOSTNAME") or os.uname().nodename).split(".", 1)[0]


def _idle(stop_path: Path) -> int:
    stopping = []
    for sig in (signal.SIGTERM, signal.SIGINT):
        signal.signal(sig, lambda *_: stopping.append(1))
    while not stopping and not stop_path.exists():
        time.sleep(0.1)
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--manifest", required=True)
    args = ap.parse_args(argv)
    manifest = json.loads(Path(args.manifest).read_text())
    if manifest.get("schema") != SCHEMA:
        raise SystemExit(f"{args.manifest}: not a {SCHEMA} manifest")
    host = short_hostname()
    local = int(os.environ.get("SLURM_LOCALID", "0"))
    slots = (manifest.get("hosts") or {}).get(host)
    if not isinstance(slots, list) or not 0 <= local < len(slots):
        raise SystemExit(f"the step has no task {local} on host {host} (hosts in the manifest: {sorted(manifest.get('hosts') or {})})")
    task = manifest["tasks"][str(slots[local])]
    if task.get("idle"):
        return _idle(Path(manifest["stop_path"]))
    os.environ.update({str(k): str(v) for k, v in task["env"].items()})
    log = task.get("log")
    if log:
        Path(log).parent.mkdir(parents=True, exist_ok=True)
        fd = os.open(log, os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o644)
        os.dup2(fd, 1)
        os.dup2(fd, 2)
        os.close(fd)
    sys.argv = [task["module"], *[str(a) for a in task.get("argv", [])]]
    try:
        runpy.run_module(task["module"], run_name="__main__", alter_sys=True)
    except SystemExit as exc:
        code = exc.code
        return int(code) if isinstance(code, int) else (0 if code is None else 1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
