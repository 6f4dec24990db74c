"""Micro-benchmarks that produce the hardware YAML the planner reads (``pipeline.py --hw hw.yaml``).

    python calibrate.py --output hw.yaml                                    # one GPU: compute, memory, decode
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29541 \
        calibrate.py --output hw.yaml                                       # plus collectives over NVLink

What is measured, all with CUDA events after warm-up (3 warm, 10 timed, median) on inputs larger than L2:
  memory_bandwidth      a 1 GiB device copy with this framework's 16-byte copy kernel
  flops_per_gpu         the tcgen05 bf16 GEMM at 8192^3
  gemm_m_half           a sweep of x[M,4096] @ W[4096,4096]^T over M, least-squares fit of eta(M) = M / (M + m_half)
  decode_layer_chain_s  CUDA-graph decode steps of a 7B-shape model at 8 and 64 rows (context 576) against the bytes they
  decode_row_layer_s    have to move (weights once + the KV of every live row) at the copy rate: what is left is the
                        latency of a layer's chain of dependent kernels and the per-row work (decode_bw_eff is 1.0)
  non_gemm_constant/..  RMSNorm + RoPE + SwiGLU + flash attention of one layer at the calibration batch
  alpha/beta (g tier)   NCCL all-reduce sweep and peer-to-peer ping-pong inside the node (needs >= 2 ranks);
                        the inter-node tiers keep the preset's values (a job is one NVSwitch node)
Rank 0 writes flat keys that ``analytic.hardware.Hardware`` accepts. Counterpart of the reference's
calibrate.py (bench_* functions :68-895, fit_alpha_beta :896, YAML emit :1196-1238).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
from typing import Callable, Dict, List, Tuple


def timed(fn: Callable[[], None], warm: int = 3, iters: int = 10) -> float:
    """Median seconds per call, CUDA events on the current stream."""
    import torch
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1) * 1e-3)
    return statistics.median(out)


def fit_alpha_beta(sizes: List[float], times: List[float], min_size: float = 1e6) -> Tuple[float, float]:
    """t = alpha + beta * bytes; beta from the large sizes, alpha from the small ones (never negative)."""
    big = [(s, t) for s, t in zip(sizes, times) if s >= min_size] or list(zip(sizes, times))
    n = len(big)
    mx, my = sum(s for s, _ in big) / n, sum(t for _, t in big) / n
    var = sum((s - mx) ** 2 for s, _ in big)
    beta = sum((s - mx) * (t - my) for s, t in big) / var if var > 0 else my / mx
    small = [(s, t) for s, t in zip(sizes, times) if s < min_size] or big[:1]
    alpha = max(0.0, statistics.median(t - beta * s for s, t in small))
    return alpha, max(beta, 1e-15)


def fit_gemm_m_half(ms: List[int], eff: List[float]) -> float:
    """Least squares for eta(M) = M / (M + m_half) in the linear form M / eta = M + m_half."""
    pts = [(m, e) for m, e in zip(ms, eff) if e > 0]
    return max(0.0, sum(m / e - m for m, e in pts) / len(pts)) if pts else 0.0


def bench_memory_bandwidth(dev) -> float:
    import ctypes
    import torch
    from rpeg_b200.ops._lib import check, lib
    n = 1 << 30
    a, b = torch.empty(n, dtype=torch.uint8, device=dev), torch.empty(n, dtype=torch.uint8, device=dev)
    s = lambda: torch.cuda.current_stream().cuda_stream
    t = timed(lambda: check(lib().rpeg_copy16(a.data_ptr(), b.data_ptr(), n, s()), "rpeg_copy16"))
    return 2 * n / t


def bench_gemm(dev) -> Dict[str, float]:
    import torch
    from rpeg_b200.ops import kernels as K
    a = torch.randn(8192, 8192, device=dev).bfloat16()
    w = torch.randn(8192, 8192, device=dev).bfloat16()
    out = torch.empty(8192, 8192, dtype=torch.bfloat16, device=dev)
    peak = 2 * 8192 ** 3 / timed(lambda: K.gemm(a, w, out=out))
    w4 = torch.randn(4096, 4096, device=dev).bfloat16()
    ms, eff = [], []
    for m in (128, 256, 512, 1024, 2048, 4096, 8192, 16384):
        x = torch.randn(m, 4096, device=dev).bfloat16()
        y = torch.empty(m, 4096, dtype=torch.bfloat16, device=dev)
        t = timed(lambda: K.gemm(x, w4, out=y))
        ms.append(m)
        eff.append(min(1.0, 2 * m * 4096 * 4096 / t / peak))
    return {"flops_per_gpu": peak, "gemm_m_half": fit_gemm_m_half(ms, eff), "sweep": dict(zip(map(str, ms), eff))}


def bench_decode(dev, hbm: float, layers: int) -> Dict[str, float]:
    import dataclasses
    import torch
    from rpeg_b200.engine.generation import Generator
    from rpeg_b200.models.llama import LlamaConfig, LlamaModel
    cfg = dataclasses.replace(LlamaConfig.llama7b(max_pos=2048), n_layers=layers)
    model = LlamaModel(cfg, dev, seed=1)
    gen = Generator(model, max_slots=64, max_seq_len=1024, kv_budget_bytes=1e12, eos_id=2)
    n, b, ctx = gen.max_slots, 64, 576
    gen.out_tok = torch.zeros((n, 2048), dtype=torch.int32, device=dev)
    gen.out_lp = torch.zeros((n, 2048), dtype=torch.float32, device=dev)
    gen.page_table.copy_(torch.arange(1, 1 + n * gen.pages_per_row, dtype=torch.int32, device=dev).view(n, -1))

    def reset():
        gen.active.fill_(1)
        gen.seq_len.fill_(ctx + 1)
        gen.pos.fill_(ctx)
        gen.gen_count.fill_(1)
        gen.token.fill_(5)

    weights = 2 * sum(int(p.numel()) for k, p in model.p.items() if k != "embed")
    kv_row = (ctx + 12) * 2 * cfg.n_layers * cfg.n_kv_heads * cfg.head_dim * 2
    times = {}
    for rows in (8, b):                       # a small and a large batch: the step's fixed and per-row parts
        reset()
        times[rows] = timed(lambda: gen._step(rows, 1.0, False, 0), warm=3, iters=20)
    t = times[b]
    kv = b * kv_row
    del gen, model
    torch.cuda.empty_cache()
    # The step costs its bytes at the copy rate (the attention kernel and, within a few per cent, the skinny GEMMs
    # stream at that rate) plus the latency of every layer's chain of dependent kernels plus per-row work:
    #   t(rows) = (weights + rows * kv_row) / hbm + layers * (chain + per_row * rows)
    per_row = ((times[b] - times[8]) - (b - 8) * kv_row / hbm) / (cfg.n_layers * (b - 8))
    per_row = max(0.0, per_row)
    chain = max(0.0, (times[8] - (weights + 8 * kv_row) / hbm) / cfg.n_layers - per_row * 8)
    # the older single factor (weight stream efficiency with everything else folded in), kept for comparison
    t_w = t - kv / hbm
    e_w = weights / hbm / t_w if t_w > 0 else 1.0
    if 3.5 * e_w < 1.0:
        e_w = (weights + kv / 3.5) / hbm / t
    return {"decode_step_s": t, "decode_step_small_s": times[8], "decode_bw_eff": 1.0, "decode_bw_eff_single_factor": min(1.0, e_w),
            "decode_layer_chain_s": chain, "decode_row_layer_s": per_row,
            "decode_step_traffic_fraction": min(1.0, (weights + kv) / hbm / t)}


def bench_non_gemm(dev, batch: int = 64, seq: int = 640) -> Dict[str, float]:
    """Seconds per layer of the non-GEMM kernels at ``batch`` sequences of ``seq`` tokens; the part that
    does not shrink with tensor parallelism (norms, residuals) is the constant, the rest the scaling."""
    import math
    import torch
    from rpeg_b200.ops import kernels as K
    d, f, H, hd = 4096, 11008, 32, 128
    T = batch * seq
    x = torch.randn(T, d, device=dev).bfloat16()
    w = torch.ones(d, device=dev).bfloat16()
    qkv = torch.randn(T, 3 * d, device=dev).bfloat16()
    gu = torch.randn(T, 2 * f, device=dev).bfloat16()
    pos = torch.arange(seq, device=dev, dtype=torch.int32).repeat(batch)
    cu = torch.arange(0, T + 1, seq, device=dev, dtype=torch.int32)
    cos_t, sin_t = K.rope_tables(seq, hd, 10000.0, dev)
    t_norm = timed(lambda: K.rmsnorm_fwd(x, w, 1e-5, residual=x, want_sum=True))
    t_rope = timed(lambda: (K.rope_(qkv, pos, cos_t, sin_t, 0, H, hd), K.rope_(qkv, pos, cos_t, sin_t, d, H, hd)))
    t_act = timed(lambda: K.swiglu_fwd(gu))
    t_attn = timed(lambda: K.flash_attn_fwd(qkv, 0, d, 2 * d, cu, seq, H, H, hd))
    return {"non_gemm_constant": 2 * t_norm, "non_gemm_scaling": t_rope + t_act + t_attn, "non_gemm_batch_cal": float(batch),
            "parts": {"rmsnorm": t_norm, "rope": t_rope, "swiglu": t_act, "flash_attn": t_attn}}


def bench_engine_terms(dev, peak: float, parts: Dict[str, float], batch: int = 64, seq: int = 640) -> Dict[str, float]:
    """The cost model's engine terms: GEMM rate held over seconds (power cap) relative to the burst rate, the rate
    attention FLOPs reach in a training mix (two forwards with recompute, one backward) relative to the sustained
    GEMM rate, and the elementwise kernels' seconds per token and layer."""
    import time
    import torch
    from rpeg_b200.ops import kernels as K
    a = torch.randn(8192, 8192, device=dev).bfloat16()
    w = torch.randn(8192, 8192, device=dev).bfloat16()
    out = torch.empty(8192, 8192, dtype=torch.bfloat16, device=dev)
    for _ in range(3):
        K.gemm(a, w, out=out)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n, t_host = 0, time.monotonic()
    e0.record()
    while time.monotonic() - t_host < 2.5:
        for _ in range(50):
            K.gemm(a, w, out=out)
        n += 50
        torch.cuda.synchronize()
    e1.record()
    torch.cuda.synchronize()
    sustained = 2 * 8192 ** 3 * n / (e0.elapsed_time(e1) * 1e-3)
    del a, w, out
    d, H, hd, s_att, b_att = 4096, 32, 128, 2048, 8
    T = b_att * s_att
    qkv = torch.randn(T, 3 * d, device=dev).bfloat16()
    cu = torch.arange(0, T + 1, s_att, device=dev, dtype=torch.int32)
    o, lse = K.flash_attn_fwd(qkv, 0, d, 2 * d, cu, s_att, H, H, hd)
    do = torch.randn_like(o)
    t_f = timed(lambda: K.flash_attn_fwd(qkv, 0, d, 2 * d, cu, s_att, H, H, hd))
    t_b = timed(lambda: K.flash_attn_bwd(qkv, 0, d, 2 * d, o, do, lse, cu, s_att, H, H, hd))
    causal_fwd_flops = T * 2.0 * s_att * d                   # what the cost model counts per layer: 2 * ctx * d per token
    att_eff = 4.0 * causal_fwd_flops / (2 * t_f + t_b) / sustained
    elementwise = (2 * parts["rmsnorm"] + parts["rope"] + parts["swiglu"]) / (batch * seq)
    return {"sustained_flops_fraction": min(1.0, sustained / peak), "attention_flops_eff": min(1.0, att_eff),
            "elementwise_s_per_token_layer": elementwise, "ffn_matrices": 3.0,
            "detail": {"sustained_flops": sustained, "flash_fwd_s": t_f, "flash_bwd_s": t_b,
                       "flash_fwd_tflops": causal_fwd_flops / t_f / 1e12, "flash_bwd_tflops": 2.5 * causal_fwd_flops / t_b / 1e12}}


def bench_collectives(dev, world: int) -> Dict[str, float]:
    """NCCL all-reduce sweep (bf16) and rank 0 <-> rank 1 ping-pong; device time, max over ranks."""
    import torch
    import torch.distributed as dist
    sizes = [256 * 1024, 512 * 1024] + [int(10 ** (6 + 0.3 * i)) // 2 * 2 for i in range(10)]
    ar_t, p2p_t = [], []
    rank = dist.get_rank()
    for nbytes in sizes:
        buf = torch.zeros(nbytes // 2, dtype=torch.bfloat16, device=dev)
        t = torch.tensor([timed(lambda: dist.all_reduce(buf))], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ar_t.append(t.item())

        def pingpong():
            if rank == 0:
                dist.send(buf, 1)
                dist.recv(buf, 1)
            elif rank == 1:
                dist.recv(buf, 0)
                dist.send(buf, 0)

        tp = torch.tensor([timed(pingpong) / 2 if rank < 2 else 0.0], device=dev, dtype=torch.float64)
        dist.all_reduce(tp, op=dist.ReduceOp.MAX)
        p2p_t.append(tp.item())
    # ring-model bytes on the wire per rank: 2 (p-1)/p * M, so the fitted beta is per wire byte as the cost model expects
    wire = [2 * (world - 1) / world * s for s in sizes]
    a_c, b_c = fit_alpha_beta(wire, ar_t)
    a_p, b_p = fit_alpha_beta([float(s) for s in sizes], p2p_t)
    big = sizes[-1]
    return {"alpha_coll_g": a_c / max(1, 2 * (world - 1)), "beta_coll_g": b_c, "alpha_p2p_g": a_p, "beta_p2p_g": b_p,
            "allreduce_busbw_gbs": 2 * (world - 1) / world * big / ar_t[-1] / 1e9, "p2p_gbs": big / p2p_t[-1] / 1e9,
            "allreduce_sweep": dict(zip(map(str, sizes), ar_t)), "p2p_sweep": dict(zip(map(str, sizes), p2p_t))}


def bench_fused_paths(dev, world: int) -> Dict[str, object]:
    """This framework's own multi-GPU kernels at their working sizes (more than one rank): the fused all-reduce +
    residual + RMSNorm of tensor-parallel decoding (microseconds per launch at 256 rows x 4096) and the gradient
    reduction of the fused data-parallel optimizer step (GB/s of peer gradient bytes entering a rank)."""
    import ctypes
    import torch
    import torch.distributed as dist
    from rpeg_b200.ops._lib import check, lib
    from rpeg_b200.parallel.symm import SymmetricBuffer
    from rpeg_b200.parallel.tp_decode_selftest import time_collectives
    out: Dict[str, object] = {"tp_decode": time_collectives(dev, world)}
    n = 256 * 1024 * 1024                                  # fp32 elements of "gradients" per rank (1 GiB)
    grads = SymmetricBuffer(n * 4, dev, None, zero=True)
    per = n // world // 64 * 64
    reduced = torch.empty(per, dtype=torch.float32, device=dev)
    sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
    rank = dist.get_rank()
    stream = torch.cuda.current_stream().cuda_stream

    def reduce_once():
        check(lib().rpeg_dp_reduce_norm(grads.ptr_array(), world, rank * per, per, 1.0, reduced.data_ptr(), sumsq.data_ptr(), stream),
              "rpeg_dp_reduce_norm")

    dist.barrier()
    t = torch.tensor([timed(reduce_once, warm=2, iters=5)], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    out["dp_reduce_s"] = float(t.item())
    out["dp_reduce_gbs"] = (world - 1) * per * 4 / float(t.item()) / 1e9
    dist.barrier()
    grads.close()
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Calibrate the planner's hardware model on this machine")
    ap.add_argument("--output", default="hw.yaml")
    ap.add_argument("--decode-layers", type=int, default=32, help="layers of the 7B-shape model used for the decode step")
    ap.add_argument("--skip", default="", help="comma list of: memory,gemm,decode,non_gemm,engine,collectives,fused")
    args = ap.parse_args(argv)
    import torch
    import torch.distributed as dist
    import yaml
    from rpeg_b200.analytic.hardware import b200_nvswitch
    skip = set(filter(None, args.skip.split(",")))
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    base = b200_nvswitch()
    hw: Dict[str, object] = {k: getattr(base, k) for k in base.field_names()}
    detail: Dict[str, object] = {}
    if rank == 0:
        if "memory" not in skip:
            hw["memory_bandwidth"] = bench_memory_bandwidth(dev)
        if "gemm" not in skip:
            g = bench_gemm(dev)
            hw["flops_per_gpu"], hw["gemm_m_half"] = g["flops_per_gpu"], g["gemm_m_half"]
            detail["gemm_efficiency_by_m"] = g["sweep"]
        if "non_gemm" not in skip:
            n = bench_non_gemm(dev)
            hw.update({k: n[k] for k in ("non_gemm_constant", "non_gemm_scaling", "non_gemm_batch_cal")})
            detail["non_gemm_parts_s"] = n["parts"]
            if "engine" not in skip and "gemm" not in skip:
                e = bench_engine_terms(dev, float(hw["flops_per_gpu"]), n["parts"])
                hw.update({k: e[k] for k in ("sustained_flops_fraction", "attention_flops_eff", "elementwise_s_per_token_layer", "ffn_matrices")})
                detail["engine_terms"] = e["detail"]
        if "decode" not in skip:
            d = bench_decode(dev, float(hw["memory_bandwidth"]), args.decode_layers)
            hw["decode_bw_eff"] = d["decode_bw_eff"]
            hw["decode_layer_chain_s"], hw["decode_row_layer_s"] = d["decode_layer_chain_s"], d["decode_row_layer_s"]
            detail["decode_step_s"] = d["decode_step_s"]
            detail["decode_step_small_s"] = d["decode_step_small_s"]
            detail["decode_bw_eff_single_factor"] = d["decode_bw_eff_single_factor"]
        hw["memory_per_gpu"] = float(torch.cuda.get_device_properties(dev).total_memory)
    if world > 1:
        dist.barrier()
        if "collectives" not in skip:
            c = bench_collectives(dev, world)
            for k in ("alpha_coll_g", "beta_coll_g", "alpha_p2p_g", "beta_p2p_g"):
                hw[k] = c[k]
            detail.update(allreduce_busbw_gbs=c["allreduce_busbw_gbs"], p2p_gbs=c["p2p_gbs"], allreduce_sweep_s=c["allreduce_sweep"],
                          p2p_sweep_s=c["p2p_sweep"])
        if "fused" not in skip:
            f = bench_fused_paths(dev, world)
            hw["tp_decode_allreduce_s"] = float(f["tp_decode"]["allreduce_rmsnorm_us"]) * 1e-6
            small = [v for k, v in f["tp_decode"].items() if k.endswith("rows_one_shot_us")]
            if small:
                hw["tp_decode_allreduce_small_s"] = float(min(small)) * 1e-6
            hw["dp_reduce_gbs"] = float(f["dp_reduce_gbs"])
            detail["fused_paths"] = f
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        out = {k: (v if isinstance(v, str) else float(v)) for k, v in hw.items()}
        with open(args.output, "w") as f:
            f.write("# written by calibrate.py on " + torch.cuda.get_device_name(dev) + f", {world} rank(s)\n")
            yaml.safe_dump(out, f, sort_keys=False)
        with open(os.path.splitext(args.output)[0] + ".detail.json", "w") as f:
            json.dump(detail, f, indent=1)
        print(json.dumps({"output": args.output, **{k: out[k] for k in ("flops_per_gpu", "memory_bandwidth", "gemm_m_half", "decode_bw_eff",
                                                                        "non_gemm_constant", "non_gemm_scaling", "alpha_coll_g", "beta_coll_g",
                                                                        "alpha_p2p_g", "beta_p2p_g", "sustained_flops_fraction",
                                                                        "attention_flops_eff", "elementwise_s_per_token_layer")}}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
