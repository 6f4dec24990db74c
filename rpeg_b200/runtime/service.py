"""Long-lived worker group that serves requests of a controller: the worker side of the request tier.

    python -m rpeg_b200.runtime.service --table toy|engine [--backend gloo|nccl]

One process per rank (per GPU with ``nccl``). Rank 0 listens on a loopback TCP port, which it publishes in its
``ready`` heartbeat; a request is one length-prefixed JSON message ``{operation, node_id, step, payload}``. Rank 0
hands it to the other ranks with ``broadcast_object_list``, every rank runs the operation of its table (the
operations may use collectives among the ranks), the per-rank results are gathered on rank 0 and sent back as
``{"ok": true, "results": [...]}`` or ``{"ok": false, "error": ...}``. A rank whose operation raised reports an
``error`` heartbeat, the group answers the request with the error and leaves: the controller decides whether the
group can be started again and brought back to its state by replaying the journal of its state-building requests.
A group whose controller closed the connection (or died) shuts itself down.

Tables: ``toy`` keeps a small CPU tensor per rank as "the model" (control-plane tests, no GPU); ``engine`` holds
``LlamaModel`` + ``AdamW`` on the rank's GPU. Operations shared by both: ``build_model``, ``load_weight_version``,
``save_weight_version``, ``lm_training_step``, ``checksum``, ``shutdown``.

Host-side failure injection (never on the device), only in the launch generation named by
``RPEG_TEST_FAIL_GENERATION`` (default 0, the first launch, so that a restarted group runs clean):
  RPEG_TEST_FAIL_OPERATION=<operation>   the request at which the chosen rank fails
  RPEG_TEST_FAIL_RANK=<r>                (default 0)
  RPEG_TEST_FAIL_MODE=exit|raise|exit_after   leave with code 3 before running it | raise inside it | leave after
                                              answering it (the group is then found dead BEFORE the next request)
Reference: the worker side of RPEG/runtime/semantic_worker.py:311-326 (injection), :5503-5872 (operation dispatch)
and the socket clients of RPEG/runtime/semantic_controller.py:423-455.
"""
from __future__ import annotations

import argparse
import json
import os
import socket
import struct
import sys
from typing import Any, Callable, Dict, List, Optional

from .control import HeartbeatStore

MAX_MESSAGE = 64 << 20


# ---------------------------------------------------------------------------------------------------- framing
def send_message(sock: socket.socket, obj: Any) -> None:
    data = json.dumps(obj).encode()
    if len(data) > MAX_MESSAGE:
        raise ValueError(f"message of {len(data)} bytes exceeds the {MAX_MESSAGE} byte limit; pass tensors by path")
    sock.sendall(struct.pack("<I", len(data)) + data)


def _recv_exact(sock: socket.socket, n: int) -> bytes:
    buf = bytearray()
    while len(buf) < n:
        chunk = sock.recv(n - len(buf))
        if not chunk:
            raise ConnectionError("peer closed the connection")
        buf += chunk
    return bytes(buf)


def recv_message(sock: socket.socket) -> Any:
    (n,) = struct.unpack("<I", _recv_exact(sock, 4))
    if n > MAX_MESSAGE:
        raise ConnectionError(f"announced message of {n} bytes exceeds the limit")
    return json.loads(_recv_exact(sock, n).decode())


# ---------------------------------------------------------------------------------------------------- operation tables
class ToyTable:
    """The "model" is ``dim`` floats per rank. A training step adds the all-reduced mean of a rank-dependent gradient,
    so the state after a sequence of requests is a deterministic function of the sequence."""

    def __init__(self, rank: int, world: int, dist):
        self.rank, self.world, self.dist = rank, world, dist
        self.w = None
        self.version: Optional[int] = None

    def build_model(self, p: Dict[str, Any]) -> Dict[str, Any]:
        import torch
        g = torch.Generator().manual_seed(int(p.get("seed", 0)))
        self.w = torch.randn(int(p.get("dim", 16)), generator=g, dtype=torch.float64)
        self.version = 0
        return {"dim": int(self.w.numel())}

    def save_weight_version(self, p: Dict[str, Any]) -> Dict[str, Any]:
        import torch
        if self.rank == 0:
            tmp = f"{p['path']}.tmp{os.getpid()}"
            torch.save({"w": self.w, "version": int(p["version"])}, tmp)
            os.replace(tmp, p["path"])
        if self.world > 1:
            self.dist.barrier()
        self.version = int(p["version"])
        return {"version": self.version}

    def load_weight_version(self, p: Dict[str, Any]) -> Dict[str, Any]:
        import torch
        blob = torch.load(p["path"], weights_only=True)
        self.w, self.version = blob["w"].clone(), int(blob["version"])
        return {"version": self.version}

    def lm_training_step(self, p: Dict[str, Any]) -> Dict[str, Any]:
        import torch
        g = torch.full_like(self.w, float(self.rank + 1) * float(p.get("scale", 1.0)))
        if self.world > 1:
            self.dist.all_reduce(g)
        self.w -= float(p.get("lr", 0.1)) * g / self.world
        return {"grad_norm": float(g.norm())}

    def checksum(self, p: Dict[str, Any]) -> Dict[str, Any]:
        return {"checksum": None if self.w is None else float(self.w.sum()), "version": self.version}


class EngineTable:
    """``LlamaModel`` + ``AdamW`` on this rank's GPU (every rank a full replica; gradients all-reduced with NCCL)."""

    def __init__(self, rank: int, world: int, dist):
        import torch
        self.rank, self.world, self.dist = rank, world, dist
        self.device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        self.model = self.opt = None
        self.version: Optional[int] = None

    def build_model(self, p: Dict[str, Any]) -> Dict[str, Any]:
        from ..engine.optimizer import AdamW
        from ..models.llama import LlamaConfig, LlamaModel
        cfg = LlamaConfig(**p["config"])
        self.model = LlamaModel(cfg, self.device, seed=int(p.get("seed", 0)), trainable=True)
        self.opt = AdamW(self.model, lr=float(p.get("lr", 1e-4)))
        self.version = 0
        return {"parameters": int(self.model.layout.total)}

    def save_weight_version(self, p: Dict[str, Any]) -> Dict[str, Any]:
        import torch
        if self.rank == 0:
            tmp = f"{p['path']}.tmp{os.getpid()}"
            torch.save({"w": self.model.w.cpu(), "version": int(p["version"])}, tmp)
            os.replace(tmp, p["path"])
        if self.world > 1:
            self.dist.barrier()
        self.version = int(p["version"])
        return {"version": self.version}

    def load_weight_version(self, p: Dict[str, Any]) -> Dict[str, Any]:
        import torch
        blob = torch.load(p["path"], weights_only=True)
        self.model.w.copy_(blob["w"].to(self.device))
        self.opt.master.copy_(self.model.w[self.opt.shard_off:self.opt.shard_off + self.opt.shard_n].float())
        self.version = int(blob["version"])
        return {"version": self.version}

    def lm_training_step(self, p: Dict[str, Any]) -> Dict[str, Any]:
        """One clipped-policy step on a synthetic rollout that is a function of ``seed`` and the rank."""
        import torch
        from ..engine import algorithms as A
        cfg = self.model.cfg
        n, s, t = int(p.get("batch", 2)), int(p.get("prompt_len", 16)), int(p.get("resp_len", 16))
        g = torch.Generator(device="cpu").manual_seed(int(p.get("seed", 0)) * 977 + self.rank)
        dev = self.device
        ro = A.Rollout(torch.randint(3, cfg.vocab, (n, s), generator=g, dtype=torch.int32).to(dev), [s] * n,
                       torch.randint(3, cfg.vocab, (n, t), generator=g, dtype=torch.int32).to(dev), [t] * n,
                       torch.zeros(n, t, device=dev), torch.ones(n, t, device=dev))
        algo = A.AlgoConfig(micro_tokens=4096, head_chunk=1024)
        ro.old_logp = A.sequence_logprobs(self.model, ro, algo)
        ro.adv = torch.randn(n, t, generator=g).to(dev)
        self.model.g.zero_()
        out = A.policy_train_step(self.model, ro, algo, denom_tokens=float(n * t * self.world))
        if self.world > 1:
            self.dist.all_reduce(self.model.g)
        self.opt.step()
        return {"loss": float(out["loss"].item()), "grad_norm": float(self.opt.grad_norm().item())}

    def checksum(self, p: Dict[str, Any]) -> Dict[str, Any]:
        return {"checksum": None if self.model is None else float(self.model.w.float().sum().item()), "version": self.version}


TABLES: Dict[str, Callable[..., Any]] = {"toy": ToyTable, "engine": EngineTable}


# ---------------------------------------------------------------------------------------------------- the server loop
def _injected(operation: str, rank: int) -> Optional[str]:
    if os.environ.get("RPEG_TEST_FAIL_OPERATION") != operation:
        return None
    if int(os.environ.get("RPEG_TEST_FAIL_RANK", "0")) != rank:
        return None
    if int(os.environ.get("RPEG_TEST_FAIL_GENERATION", "0")) != int(os.environ.get("RPEG_LAUNCH_GENERATION", "0")):
        return None
    return os.environ.get("RPEG_TEST_FAIL_MODE", "exit")


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--table", default="toy", choices=sorted(TABLES))
    ap.add_argument("--backend", default="gloo", choices=("gloo", "nccl"))
    ap.add_argument("--collective-timeout", type=float, default=30.0)
    args = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    group = os.environ.get("RPEG_GROUP_ID", "group")
    store = HeartbeatStore(os.environ.get("RPEG_HEARTBEAT_DIR", "heartbeats"))
    store.write(group, rank, "starting")
    listener = conn = None
    try:
        import datetime

        import torch
        import torch.distributed as dist
        if args.backend == "nccl":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        if world > 1:
            dist.init_process_group(args.backend, timeout=datetime.timedelta(seconds=args.collective_timeout))
        table = TABLES[args.table](rank, world, dist)
        if rank == 0:
            listener = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
            listener.bind(("127.0.0.1", 0))
            listener.listen(1)
            store.write(group, rank, "ready", message=json.dumps({"port": listener.getsockname()[1]}))
            conn, _ = listener.accept()
        else:
            store.write(group, rank, "ready")
        while True:
            box: List[Any] = [None]
            if rank == 0:
                try:
                    box[0] = recv_message(conn)
                except (ConnectionError, OSError):
                    # the controller is gone (it closed the connection or died): nobody will ever send a request again,
                    # so the group leaves in an orderly way instead of lingering on its GPUs
                    box[0] = {"operation": "shutdown", "orphaned": True}
            if world > 1:
                dist.broadcast_object_list(box, src=0)
            req = box[0]
            op, payload = req["operation"], req.get("payload") or {}
            if op == "shutdown":
                if rank == 0 and not req.get("orphaned"):
                    send_message(conn, {"ok": True, "results": []})
                break
            mode = _injected(op, rank)
            if mode == "exit":
                os._exit(3)                            # between requests: nothing of this rank is in flight
            store.write(group, rank, "running", step=req.get("step"), message=op)
            err = None
            try:
                if mode == "raise":
                    raise RuntimeError(f"injected failure in {op}")
                fn = getattr(table, op, None)
                if fn is None or op.startswith("_"):
                    raise ValueError(f"unknown operation {op!r}")
                result = fn(payload)
            except Exception as exc:
                err, result = f"{type(exc).__name__}: {exc}", None
            mine = {"rank": rank, "result": result, "error": err}
            if world > 1:
                gathered: Optional[List[Any]] = [None] * world if rank == 0 else None
                dist.gather_object(mine, gathered, dst=0)
                flag = [None if rank else next((g["error"] for g in gathered if g["error"]), None)]
                dist.broadcast_object_list(flag, src=0)
                failed = flag[0]
            else:
                gathered, failed = [mine], err
            if rank == 0:
                if failed:
                    send_message(conn, {"ok": False, "error": failed, "results": gathered})
                else:
                    send_message(conn, {"ok": True, "results": [g["result"] for g in gathered]})
            if failed:
                store.write(group, rank, "error" if err else "stopped", message=err or f"a peer failed in {op}")
                return 1 if err else 4
            store.write(group, rank, "ready", step=req.get("step"))
            if mode == "exit_after":
                os._exit(3)
        store.write(group, rank, "finished")
        if world > 1:
            dist.destroy_process_group()
        return 0
    except Exception as exc:
        store.write(group, rank, "error", message=f"{type(exc).__name__}: {exc}")
        return 1
    finally:
        for s in (conn, listener):
            if s is not None:
                s.close()


if __name__ == "__main__":
    sys.exit(main())
