"""Control plane: heartbeat files that every rank process writes and the controller reads.

A rank reports ``starting | ready | running | error | stopping | stopped | finished`` with a
monotonically increasing sequence number, its pid and an optional message. Files are replaced
atomically (tmp + rename), reads retry over the short window in which a shared filesystem may show
neither the old nor the new file. The controller waits for a whole group to reach a state with a
deadline and fails fast as soon as any rank reports ``error`` or its process is gone, which is how a
failed rank is learnt about *on the host* before the next device launch.
Reference: RPEG/runtime/control.py:23-209.
"""
from __future__ import annotations

import errno
import json
import os
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Callable, Dict, Iterable, List, Optional

from .errors import RuntimeExecutionError
from .io import atomic_write_text

STATES = ("starting", "ready", "running", "error", "stopping", "stopped", "finished")
TERMINAL = ("error", "stopped", "finished")
_TRANSIENT = (errno.ENOENT, errno.ESTALE, errno.EAGAIN, errno.EBUSY)


@dataclass
class Heartbeat:
    worker_id: str
    rank: int
    state: str
    timestamp: float = field(default_factory=time.time)
    sequence: int = 0
    pid: int = field(default_factory=os.getpid)
    hostname: str = field(default_factory=lambda: os.uname().nodename)
    message: Optional[str] = None
    step: Optional[int] = None

    def __post_init__(self):
        if self.state not in STATES:
            raise ValueError(f"unknown heartbeat state {self.state!r}")


class HeartbeatStore:
    def __init__(self, root):
        self.root = Path(root)
        self.root.mkdir(parents=True, exist_ok=True)
        self._seq: Dict[str, int] = {}

    def path(self, worker_id: str, rank: int) -> Path:
        return self.root / f"{worker_id.replace('/', '_')}.rank{rank}.json"

    def write(self, worker_id: str, rank: int, state: str, message: Optional[str] = None, step: Optional[int] = None) -> Heartbeat:
        key = f"{worker_id}:{rank}"
        self._seq[key] = self._seq.get(key, 0) + 1
        hb = Heartbeat(worker_id, rank, state, sequence=self._seq[key], message=message, step=step)
        atomic_write_text(self.path(worker_id, rank), json.dumps(asdict(hb)))
        return hb

    def read(self, worker_id: str, rank: int, retries: int = 5, delay_s: float = 0.01) -> Optional[Heartbeat]:
        p = self.path(worker_id, rank)
        for attempt in range(retries):
            try:
                return Heartbeat(**json.loads(p.read_text()))
            except FileNotFoundError:
                return None
            except OSError as exc:
                if exc.errno not in _TRANSIENT or attempt == retries - 1:
                    raise
            except json.JSONDecodeError:
                if attempt == retries - 1:
                    raise
            time.sleep(delay_s)
        return None

    def read_group(self, worker_id: str, world: int) -> List[Optional[Heartbeat]]:
        return [self.read(worker_id, r) for r in range(world)]


class ControlPlane:
    def __init__(self, store: HeartbeatStore, poll_s: float = 0.02):
        self.store, self.poll_s = store, poll_s

    def wait_for_state(self, worker_id: str, world: int, states: Iterable[str], timeout_s: float,
                       alive: Optional[Callable[[int], bool]] = None) -> List[Heartbeat]:
        """Block until every rank reports one of ``states``. Raises as soon as a rank reports ``error``
        (unless waited for), a rank's process is gone (``alive(rank)`` false) or the deadline passes."""
        want = set(states)
        deadline = time.monotonic() + timeout_s
        while True:
            beats = self.store.read_group(worker_id, world)
            for r, hb in enumerate(beats):
                if hb is not None and hb.state == "error" and "error" not in want:
                    raise RuntimeExecutionError(f"{worker_id} rank {r} reported an error: {hb.message}")
                if alive is not None and not alive(r) and (hb is None or hb.state not in TERMINAL):
                    raise RuntimeExecutionError(f"{worker_id} rank {r} exited without reporting (last state: "
                                                f"{None if hb is None else hb.state})")
            if all(hb is not None and hb.state in want for hb in beats):
                return beats  # type: ignore[return-value]
            if time.monotonic() > deadline:
                seen = {r: (None if hb is None else hb.state) for r, hb in enumerate(beats)}
                raise RuntimeExecutionError(f"{worker_id}: timed out after {timeout_s:.1f}s waiting for {sorted(want)}; states={seen}")
            time.sleep(self.poll_s)

    def assert_healthy(self, worker_id: str, world: int, alive: Optional[Callable[[int], bool]] = None,
                       stale_after_s: Optional[float] = None) -> None:
        """Checked by the controller before every request it sends to a group."""
        now = time.time()
        for r, hb in enumerate(self.store.read_group(worker_id, world)):
            if hb is None:
                raise RuntimeExecutionError(f"{worker_id} rank {r} has no heartbeat")
            if hb.state == "error":
                raise RuntimeExecutionError(f"{worker_id} rank {r} reported an error: {hb.message}")
            if alive is not None and not alive(r):
                raise RuntimeExecutionError(f"{worker_id} rank {r} is no longer running")
            if stale_after_s is not None and hb.state == "running" and now - hb.timestamp > stale_after_s:
                raise RuntimeExecutionError(f"{worker_id} rank {r} heartbeat is {now - hb.timestamp:.1f}s old")
