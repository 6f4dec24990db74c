"""JSONL runtime trace: one event per line,
``{run_id, node_id, event in {start, finish, replay, recover}, status, timestamp, worker_id, step,
counters}``. Writers append and flush every event so a trace survives a crash and can drive
recovery (reference: RPEG/runtime/trace.py:59-111, RPEG/runtime/recovery.md:56-71)."""
from __future__ import annotations

import json
import threading
import time
from pathlib import Path
from typing import Any, Dict, Iterable, List, Optional

EVENTS = ("start", "finish", "replay", "recover")


class RuntimeTraceWriter:
    def __init__(self, path, run_id: str, append: bool = False):
        self.path = Path(path)
        self.path.parent.mkdir(parents=True, exist_ok=True)
        self.run_id = run_id
        self._lock = threading.Lock()
        self._f = open(self.path, "a" if append else "w", buffering=1)

    def emit(self, node_id: str, event: str, *, status: str = "ok", worker_id: Optional[str] = None,
             step: Optional[int] = None, counters: Optional[Dict[str, Any]] = None, timestamp: Optional[float] = None,
             **extra) -> dict:
        if event not in EVENTS:
            raise ValueError(f"unknown trace event {event!r}")
        rec = {"run_id": self.run_id, "node_id": node_id, "event": event, "status": status,
               "timestamp": time.time() if timestamp is None else timestamp, "worker_id": worker_id, "step": step,
               "counters": counters or {}}
        rec.update(extra)
        with self._lock:
            self._f.write(json.dumps(rec, sort_keys=True) + "\n")
        return rec

    def close(self) -> None:
        with self._lock:
            if not self._f.closed:
                self._f.flush()
                self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def read_trace(path) -> List[dict]:
    out = []
    with open(path) as f:
        for line in f:
            line = line.strip()
            if line:
                out.append(json.loads(line))
    return out
