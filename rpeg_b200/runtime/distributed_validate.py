"""Sanity worker for a freshly launched group of ranks:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29581 \
        -m rpeg_b200.runtime.distributed_validate [--backend nccl|gloo] [--output report.json]

Every rank joins the process group, all-reduces a rank-dependent vector, all-gathers its hostname and
device and (nccl) checks a peer-memory round trip through a symmetric buffer. Rank 0 prints
``rpeg.distributed_validation.v1`` with the expected and observed sums. Works on CPU with gloo, which
is how the launch path is tested without GPUs. Reference: RPEG/runtime/distributed_validate.py:22-76.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional

SCHEMA = "rpeg.distributed_validation.v1"


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default=None, choices=(None, "nccl", "gloo"))
    ap.add_argument("--output", default=None)
    args = ap.parse_args(argv)
    import torch
    import torch.distributed as dist
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    backend = args.backend or ("nccl" if torch.cuda.is_available() else "gloo")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29581")
    if backend == "nccl":
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    x = torch.arange(1024, dtype=torch.float32, device=dev) * (rank + 1)
    dist.all_reduce(x)
    expect = float(torch.arange(1024, dtype=torch.float64).sum() * world * (world + 1) / 2)
    info: List[Optional[dict]] = [None] * world
    me = {"rank": rank, "host": os.uname().nodename, "device": torch.cuda.get_device_name(dev) if backend == "nccl" else "cpu", "local_rank": local}
    dist.all_gather_object(info, me)
    peer_ok = None
    if backend == "nccl" and world > 1:
        from ..ops._lib import check, lib
        from ..parallel.symm import SymmetricBuffer
        sym = SymmetricBuffer(4096, dev)
        sym.tensor(torch.float32).fill_(float(rank))
        torch.cuda.synchronize()
        dist.barrier()
        got = torch.empty(1024, dtype=torch.float32, device=dev)
        nxt = (rank + 1) % world
        check(lib().rpeg_copy16(sym.peer_ptrs[nxt], got.data_ptr(), 4096, torch.cuda.current_stream().cuda_stream), "rpeg_copy16")
        flag = torch.tensor([float(bool((got == float(nxt)).all()))], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        peer_ok = bool(flag.item() == 1.0)
        dist.barrier()
        sym.close()
    ok = abs(float(x.double().sum()) - expect) <= 1e-6 * expect and peer_ok is not False
    rep = {"schema_version": SCHEMA, "ok": ok, "backend": backend, "world": world, "all_reduce_sum": float(x.double().sum()),
           "expected_sum": expect, "peer_memory_ok": peer_ok, "ranks": info}
    if rank == 0:
        if args.output:
            with open(args.output, "w") as f:
                json.dump(rep, f, indent=1)
        print(json.dumps(rep))
    dist.barrier()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
