"""Micro-benchmark of one decode step of the paged-KV generator.

    python -m rpeg_b200.engine.decode_bench --slots 64 --ctx 512,1024 --batches 8,32,64

Fills every slot with a synthetic context of ``ctx`` tokens, then times ``iters`` graph replays of the
decode step (all GEMMs, rope, KV append, paged attention, sampling, bookkeeping) with CUDA events.
Prints one JSON line per (batch, ctx) with the measured time and the memory-traffic floor
(weights once + the KV of every live row) at the given HBM bandwidth. ``--layers`` shrinks the model
so a profiler capture of single kernels stays small; ``--no-graphs`` launches kernels one by one.
The numbers feed ``decode_bw_eff`` of the planner's cost model.

Under ``torch.distributed.run`` with N ranks the step is the tensor-parallel one (``models.tp_decode.TPDecodeModel``
over all ranks, every rank holding 1/N of the weights and KV heads of all rows); the traffic floor is then per rank.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--slots", type=int, default=64)
    ap.add_argument("--max-len", type=int, default=2048)
    ap.add_argument("--ctx", default="512,1024")
    ap.add_argument("--batches", default="8,32,64")
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--hbm-gbs", type=float, default=6528.7)
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--group-attention", action="store_true", help="with --share: score each group's queries against the shared "
                    "keys in one pass (the group kernel) instead of relying on L2 hits")
    ap.add_argument("--group-tc", action="store_true", help="with --group-attention: the tcgen05 group kernel instead of the CUDA-core one")
    ap.add_argument("--share", default="", help="K:S - groups of K consecutive rows alias the KV pages of their first S tokens "
                    "(K samples of one prompt), to measure what the shared pages save")
    ap.add_argument("--shard", type=int, default=1, help="on one GPU: give the model 1/N of the heads and of d_ff, i.e. the "
                    "matrix shapes a rank of N-way tensor parallelism works on (no collectives), to see the per-kernel floor")
    args = ap.parse_args(argv)

    from ..models.llama import LlamaConfig, LlamaModel
    from ..ops import kernels as K
    from .generation import Generator

    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    cfg = dataclasses.replace(LlamaConfig.llama7b(max_pos=4096), n_layers=args.layers)
    if args.shard > 1:
        cfg = dataclasses.replace(cfg, n_heads=cfg.n_heads // args.shard, n_kv_heads=cfg.n_kv_heads // args.shard,
                                  d_ff=cfg.d_ff // args.shard // 8 * 8)
    model = LlamaModel(cfg, dev, seed=1)
    whole = model
    if world > 1:
        import torch.distributed as dist
        from ..models.tp_decode import TPDecodeModel
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        model = TPDecodeModel(whole, None, max_batch=args.slots)
    gen = Generator(model, max_slots=args.slots, max_seq_len=args.max_len, kv_budget_bytes=1e12, eos_id=2,
                    use_graphs=not args.no_graphs)
    n = gen.max_slots
    gen.out_tok = torch.zeros((n, 4096), dtype=torch.int32, device=dev)
    gen.out_lp = torch.zeros((n, 4096), dtype=torch.float32, device=dev)
    gen.page_table.copy_(torch.arange(1, 1 + n * gen.pages_per_row, dtype=torch.int32, device=dev).view(n, -1))
    if args.share:
        k_share, s_share = (int(x) for x in args.share.split(":"))
        shared_pages = s_share // 64
        leader = (torch.arange(n, device=dev) // k_share) * k_share
        gen.page_table[:, :shared_pages] = gen.page_table[leader, :shared_pages]
        if args.group_attention:
            if k_share > gen.GROUP_MAX:
                raise SystemExit(f"--group-attention handles groups of at most {gen.GROUP_MAX} rows")
            gen.group_attention = True
            gen.group_min_batch = 0
            gen.group_tc = bool(args.group_tc)
            n_groups = n // k_share
            gen.group_rows.fill_(-1)
            gen.group_rows[:n_groups, :k_share] = torch.arange(n_groups * k_share, dtype=torch.int32, device=dev).view(n_groups, k_share)
            gen.group_shared[:n_groups] = shared_pages * 64
            gen.row_key0[: n_groups * k_share] = shared_pages * 64
    weight_bytes = 2 * sum(int(t.numel()) for name, t in whole.p.items() if name != "embed" and not name.startswith("scalar_head")) // world
    kv_per_token = 2 * cfg.n_layers * cfg.n_kv_heads * cfg.head_dim * 2 // world

    def reset(b: int, ctx: int) -> None:
        gen.active.zero_()
        gen.active[:b] = 1
        gen.seq_len.fill_(ctx + 1)
        gen.pos.fill_(ctx)
        gen.gen_count.fill_(1)
        gen.token.fill_(5)

    for b in (int(x) for x in args.batches.split(",")):
        if b > n:
            continue
        for ctx in (int(x) for x in args.ctx.split(",")):
            if ctx + args.iters + 8 > args.max_len:
                continue
            reset(b, ctx)
            for _ in range(3):
                gen._step(b, 1.0, False, 0)
            reset(b, ctx)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.iters):
                gen._step(b, 1.0, False, 0)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / args.iters
            floor_ms = (weight_bytes + b * (ctx + args.iters / 2) * kv_per_token) / (args.hbm_gbs * 1e9) * 1e3
            if rank == 0:
                print(json.dumps({"batch": b, "ctx": ctx, "layers": cfg.n_layers, "tp": world, "ms_per_step": round(ms, 4),
                                  "tokens_per_s": round(b / ms * 1e3, 1), "traffic_floor_ms": round(floor_ms, 4),
                                  "fraction_of_floor": round(floor_ms / ms, 4), "graphs": not args.no_graphs}), flush=True)
    K.check_status()
    if world > 1:
        model.comm.close()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
