"""Micro-benchmark of one training microbatch (policy loss, forward + backward) and of the forward-only
pass used for reference log-probs:

    python -m rpeg_b200.engine.train_bench --layers 32 --rows 16 --seq 1024 --iters 3

Builds a 7B-shape model with ``--layers`` decoder layers, a synthetic rollout of ``--rows`` sequences
of ``--seq`` tokens (half prompt, half response) and times ``policy_train_step`` and
``sequence_logprobs`` with CUDA events. Prints one JSON line with milliseconds, tokens/s and the
achieved model TFLOP/s (6 x params x tokens for training, + one more forward under full recompute;
attention FLOPs are counted separately as causal 4 x d x S/2 per token and layer) against the given
GEMM peak. A small ``--layers`` keeps a profiler capture of single kernels short.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import sys

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--rows", type=int, default=16)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--recompute", default="full", choices=("full", "none"))
    ap.add_argument("--micro-tokens", type=int, default=16384)
    ap.add_argument("--peak-tflops", type=float, default=1366.6)
    args = ap.parse_args(argv)
    from ..models.llama import LlamaConfig, LlamaModel
    from ..ops import _lib
    from ..ops import kernels as K
    from . import algorithms as A

    dev = torch.device("cuda:0")
    cfg = dataclasses.replace(LlamaConfig.llama7b(max_pos=max(4096, args.seq)), n_layers=args.layers)
    model = LlamaModel(cfg, dev, trainable=True, recompute=args.recompute, seed=1)
    N, S = args.rows, args.seq // 2
    T = args.seq - S
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(3, cfg.vocab, (N, S), generator=g, dtype=torch.int32).to(dev)
    resp = torch.randint(3, cfg.vocab, (N, T), generator=g, dtype=torch.int32).to(dev)
    ro = A.Rollout(prompts, [S] * N, resp, [T] * N, torch.zeros((N, T), device=dev), torch.ones((N, T), device=dev))
    ro.adv = torch.randn((N, T), generator=g).to(dev)
    algo = A.AlgoConfig(kl_coef=0.04, micro_tokens=args.micro_tokens, head_chunk=8192)
    ro.ref_logp = A.sequence_logprobs(model, ro, algo)
    ro.old_logp = ro.ref_logp.clone()

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        n0 = _lib.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.iters, (_lib.launch_count() - n0) // args.iters

    def train():
        model.zero_grad()
        A.policy_train_step(model, ro, algo)

    ms_train, l_train = timed(train)
    ms_fwd, l_fwd = timed(lambda: A.sequence_logprobs(model, ro, algo))
    K.check_status()
    tokens = N * args.seq
    n_mat = args.layers * (4 * cfg.d_model ** 2 + 3 * cfg.d_model * cfg.d_ff)
    head = cfg.vocab * cfg.d_model
    attn_fwd = args.layers * 4 * cfg.d_model * (args.seq / 2) * tokens          # QK^T and PV, causal
    f_fwd = 2 * n_mat * tokens + 2 * head * N * T + attn_fwd
    f_train = (4 if args.recompute == "full" else 3) * (2 * n_mat * tokens) + 3 * 2 * head * N * T \
        + (4.5 if args.recompute == "full" else 3.5) * attn_fwd
    print(json.dumps({
        "layers": args.layers, "rows": N, "seq": args.seq, "tokens": tokens, "recompute": args.recompute,
        "train_ms": round(ms_train, 3), "train_tokens_per_s": round(tokens / ms_train * 1e3, 1), "train_launches": l_train,
        "train_tflops": round(f_train / ms_train / 1e9, 1), "train_fraction_of_peak": round(f_train / ms_train / 1e9 / args.peak_tflops, 4),
        "forward_ms": round(ms_fwd, 3), "forward_tflops": round(f_fwd / ms_fwd / 1e9, 1),
        "forward_fraction_of_peak": round(f_fwd / ms_fwd / 1e9 / args.peak_tflops, 4), "forward_launches": l_fwd,
        "peak_tflops": args.peak_tflops}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
