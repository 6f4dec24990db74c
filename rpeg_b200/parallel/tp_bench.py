"""Benchmark of the fused row-parallel linear against GEMM + NCCL, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29591 \\
        -m rpeg_b200.parallel.tp_bench --rows 16384 --out-features 4096 --in-features 11008

``--in-features`` is the full contraction size (each rank holds 1 / world of it). Both arms are timed on the
device with CUDA events (3 warm-up, 10 timed, median; max over ranks); between iterations the inputs
alternate between two buffers larger than L2 in total. Prints one JSON line with the times, the
roofline target = max(FLOPs / GEMM peak, NVLink bytes / link bandwidth) and achieved / target.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist


def bench_reshard(args, rank: int, world: int, dev) -> int:
    """Llama-7B weights from the training layout's tensor-parallel shards to full replicas (and back)."""
    from ..models.llama import LlamaConfig
    from ..ops import kernels as K
    from .reshard import Layout, ReshardExecutor
    cfg = LlamaConfig.llama7b()
    rows = []
    for src_l, dst_l in ((Layout(1, 1, world), Layout(world, 1, 1)), (Layout(world, 1, 1), Layout(1, 1, world))):
        ex = ReshardExecutor(cfg, src_l, dst_l, dev)
        ex.source().normal_()
        for _ in range(2):
            ex.run()
        ts = []
        for _ in range(args.iters):
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            ex.run()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) * 1e-3], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ts.append(t.item())
        K.check_status()
        t = statistics.median(ts)
        rows.append({"src": f"dp{src_l.dp}xtp{src_l.tp}", "dst": f"dp{dst_l.dp}xtp{dst_l.tp}", "us": round(t * 1e6, 1), "launches": len(ex.plan),
                     "bytes_per_rank": ex.bytes_in, "remote_bytes_per_rank": ex.bytes_remote,
                     "remote_gbs": round(ex.bytes_remote / t / 1e9, 1), "link_fraction": round(ex.bytes_remote / t / 1e9 / args.link_gbs, 3)})
        dist.barrier()
        ex.close()
    if rank == 0:
        print(json.dumps({"mode": "reshard", "model": "llama7b", "world": world, "transitions": rows}))
    dist.barrier()
    dist.destroy_process_group()
    return 0


def bench_column(args, rank: int, world: int, dev) -> int:
    """All-gather of the activation rows + GEMM against NCCL all-gather + GEMM."""
    from ..ops import kernels as K
    from .tp import ColumnParallelLinear
    n_loc = args.out_features // world // 8 * 8
    w = (torch.randn(n_loc, args.in_features, device=dev) * 0.02).bfloat16()
    per = args.rows // world
    shards = [torch.randn(per, args.in_features, device=dev).bfloat16() for _ in range(2)]
    layer = ColumnParallelLinear(w, max_rows=args.rows, device=dev)

    def fused(i):
        layer.input_rows(args.rows).copy_(shards[i % 2])          # in a model the producer writes here directly
        layer.forward(args.rows)

    def timed(fn):
        for i in range(3):
            fn(i)
        out = []
        for i in range(args.iters):
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn(i)
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) * 1e-3], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            out.append(t.item())
        return statistics.median(out)

    t_fused = timed(fused)
    K.check_status()
    t_unfused = timed(lambda i: layer.forward_unfused(shards[i % 2]))
    full = torch.randn(args.rows, args.in_features, device=dev).bfloat16()
    t_gemm = timed(lambda i: K.gemm(full, w))
    t_copy = timed(lambda i: layer.input_rows(args.rows).copy_(shards[i % 2]))
    flops = 2.0 * args.rows * n_loc * args.in_features
    link_bytes = (world - 1) / world * args.rows * args.in_features * 2               # rows arriving at one GPU
    target = max(flops / (args.peak_tflops * 1e12), link_bytes / (args.link_gbs * 1e9))
    if rank == 0:
        print(json.dumps({"mode": "column", "world": world, "rows": args.rows, "n_per_rank": n_loc, "k": args.in_features,
                          "fused_ms": round(t_fused * 1e3, 4), "fused_without_input_copy_ms": round((t_fused - t_copy) * 1e3, 4),
                          "nccl_all_gather_plus_gemm_ms": round(t_unfused * 1e3, 4), "gemm_only_ms": round(t_gemm * 1e3, 4),
                          "speedup_vs_unfused": round(t_unfused / t_fused, 3), "roofline_target_ms": round(target * 1e3, 4),
                          "achieved_over_target": round(target / (t_fused - t_copy), 4),
                          "fused_tflops": round(flops / (t_fused - t_copy) / 1e12, 1)}))
    dist.barrier()
    layer.close()
    dist.destroy_process_group()
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--out-features", type=int, default=4096)
    ap.add_argument("--in-features", type=int, default=11008)
    ap.add_argument("--all-reduce", action="store_true")
    ap.add_argument("--mode", default="row", choices=("row", "column", "reshard"),
                    help="row: GEMM + reduce-scatter (in-features split); column: all-gather + GEMM (out-features split)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--peak-tflops", type=float, default=1608.7)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    args = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29591")
    dist.init_process_group("nccl", device_id=dev)
    from ..ops import kernels as K
    from .tp import ColumnParallelLinear, RowParallelLinear
    if args.mode == "column":
        return bench_column(args, rank, world, dev)
    if args.mode == "reshard":
        return bench_reshard(args, rank, world, dev)
    kp = args.in_features // world // 8 * 8
    w = (torch.randn(args.out_features, kp, device=dev) * 0.02).bfloat16()
    xs = [torch.randn(args.rows, kp, device=dev).bfloat16() for _ in range(2)]
    layer = RowParallelLinear(w, max_rows=args.rows, device=dev, all_reduce=args.all_reduce)

    def timed(fn):
        for i in range(3):
            fn(xs[i % 2])
        out = []
        for i in range(args.iters):
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn(xs[i % 2])
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) * 1e-3], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            out.append(t.item())
        return statistics.median(out)

    t_fused = timed(layer.forward)
    K.check_status()
    t_unfused = timed(layer.forward_unfused)
    t_gemm = timed(lambda x: K.gemm(x, w))
    flops = 2.0 * args.rows * args.out_features * kp
    factor = 2.0 if args.all_reduce else 1.0
    link_bytes = factor * (world - 1) / world * args.rows * args.out_features * 2           # bf16 partials leaving one GPU
    target = max(flops / (args.peak_tflops * 1e12), link_bytes / (args.link_gbs * 1e9))
    if rank == 0:
        print(json.dumps({"world": world, "rows": args.rows, "n": args.out_features, "k_per_rank": kp, "all_reduce": args.all_reduce,
                          "fused_ms": round(t_fused * 1e3, 4), "gemm_plus_nccl_ms": round(t_unfused * 1e3, 4),
                          "gemm_only_ms": round(t_gemm * 1e3, 4), "speedup_vs_unfused": round(t_unfused / t_fused, 3),
                          "roofline_target_ms": round(target * 1e3, 4), "achieved_over_target": round(target / t_fused, 4),
                          "fused_tflops": round(flops / t_fused / 1e12, 1), "link_gbs_out": round(link_bytes / t_fused / 1e9, 1)}))
    dist.barrier()
    layer.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
