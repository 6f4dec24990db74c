"""Collective benchmark over the node's GPUs, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29571 \
        -m rpeg_b200.runtime.collective_benchmark --sizes 1e6,1e7,1e8,1e9 --output coll.json

Times, on the device (CUDA events, max over ranks, 3 warm-up + 10 timed iterations):
  nccl_all_reduce        bf16 all-reduce                                 (bus bandwidth 2(p-1)/p * bytes / t)
  nccl_reduce_scatter    bf16 reduce-scatter
  nccl_all_gather        bf16 all-gather
  peer_pull_reduce       this framework's reduce kernel: every rank pulls its shard of all peers' fp32
                         buffers over NVLink and sums them (the gradient half of the fused optimizer step)
  peer_copy              rank r reads 1/p of rank (r+1)'s buffer with the 16-byte copy kernel
Output schema ``rpeg.collective_benchmark.v1``. Reference: RPEG/runtime/collective_benchmark.py:45-165.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
from typing import Callable, Dict, List, Optional

SCHEMA = "rpeg.collective_benchmark.v1"


def _timed(fn: Callable[[], None], dist, dev, warm: int = 3, iters: int = 10) -> float:
    import torch
    for _ in range(warm):
        fn()
    out = []
    for _ in range(iters):
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e-3], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out.append(t.item())
    return statistics.median(out)


def large_message_gate(rows: List[Dict[str, float]], min_gbps: float) -> Dict[str, object]:
    """The all-reduce bus bandwidth of the LARGEST message against a floor: a job on a node whose NVLink fabric is
    degraded should fail here, before it trains (reference: ``--min-large-message-gbps`` of
    RPEG/runtime/collective_benchmark.py:125-164)."""
    if not rows:
        return {"ok": False, "min_large_message_gbps": float(min_gbps), "measured_gbps": None, "bytes": None}
    big = max(rows, key=lambda r: r.get("bytes", 0))
    got = float(big.get("nccl_all_reduce_busbw_gbs", 0.0))
    return {"ok": got >= float(min_gbps), "min_large_message_gbps": float(min_gbps), "measured_gbps": got, "bytes": int(big.get("bytes", 0))}


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="1e6,1e7,1e8,1e9", help="bytes per rank, comma separated")
    ap.add_argument("--output", default=None)
    ap.add_argument("--min-large-message-gbps", type=float, default=0.0,
                    help="exit 2 when the all-reduce bus bandwidth of the largest message is below this (GB/s)")
    args = ap.parse_args(argv)
    import torch
    import torch.distributed as dist
    from ..ops import kernels as K
    from ..ops._lib import check, lib
    from ..parallel.symm import SymmetricBuffer
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    rows: List[Dict[str, float]] = []
    stream = lambda: torch.cuda.current_stream().cuda_stream
    for size in (int(float(s)) for s in args.sizes.split(",")):
        n = size // (4 * world * 4) * (4 * world)          # fp32 elements, divisible by world and by 4 per shard
        nb = n * 4
        x16 = torch.zeros(nb // 2, dtype=torch.bfloat16, device=dev)
        shard16 = torch.zeros(nb // 2 // world, dtype=torch.bfloat16, device=dev)
        row: Dict[str, float] = {"bytes": nb, "world": world}
        t = _timed(lambda: dist.all_reduce(x16), dist, dev)
        row["nccl_all_reduce_s"], row["nccl_all_reduce_busbw_gbs"] = t, 2 * (world - 1) / world * nb / t / 1e9
        t = _timed(lambda: dist.reduce_scatter_tensor(shard16, x16), dist, dev)
        row["nccl_reduce_scatter_s"], row["nccl_reduce_scatter_busbw_gbs"] = t, (world - 1) / world * nb / t / 1e9
        t = _timed(lambda: dist.all_gather_into_tensor(x16, shard16), dist, dev)
        row["nccl_all_gather_s"], row["nccl_all_gather_busbw_gbs"] = t, (world - 1) / world * nb / t / 1e9
        sym = SymmetricBuffer(nb, dev, zero=True)
        per = n // world
        red = torch.empty(per, dtype=torch.float32, device=dev)
        ss = torch.zeros(1, dtype=torch.float32, device=dev)
        t = _timed(lambda: check(lib().rpeg_dp_reduce_norm(sym.ptr_array(), world, rank * per, per, 1.0, red.data_ptr(), ss.data_ptr(),
                                                           stream()), "rpeg_dp_reduce_norm"), dist, dev)
        row["peer_pull_reduce_s"], row["peer_pull_reduce_busbw_gbs"] = t, (world - 1) / world * nb / t / 1e9
        src = sym.peer_ptrs[(rank + 1) % world]
        dst = torch.empty(per, dtype=torch.float32, device=dev)
        t = _timed(lambda: check(lib().rpeg_copy16(src, dst.data_ptr(), per * 4, stream()), "rpeg_copy16"), dist, dev)
        row["peer_copy_s"], row["peer_copy_gbs"] = t, per * 4 / t / 1e9
        K.check_status()
        torch.cuda.synchronize()
        dist.barrier()
        sym.close()
        rows.append(row)
    gate = large_message_gate(rows, args.min_large_message_gbps)
    if rank == 0:
        rep = {"schema_version": SCHEMA, "world": world, "device": torch.cuda.get_device_name(dev), "rows": rows, "gate": gate}
        if args.output:
            with open(args.output, "w") as f:
                json.dump(rep, f, indent=1)
        print(json.dumps(rep))
    dist.barrier()
    dist.destroy_process_group()
    return 0 if gate["ok"] else 2


if __name__ == "__main__":
    sys.exit(main())
