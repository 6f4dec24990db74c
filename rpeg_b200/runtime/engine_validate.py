"""Engine smoke worker: does this machine train, generate and checkpoint with the native engine?

    python -m rpeg_b200.runtime.engine_validate --json                                   # one GPU, tiny model
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29513 \\
        -m rpeg_b200.runtime.engine_validate --layers 4 --hidden 1024 --ffn 2816 --ppo-exercise --checkpoint-dir /tmp/ck

Run before a long job (the generated Slurm file can call it after the preflight). One process per GPU; with more
than one rank the model is data parallel over all ranks (weights and gradients in symmetric memory, fused optimizer
step). Checks, each reported as ``{name, ok, detail}``:

  build          model + optimizer at the requested size; the kernel library answers
  train_step     random tokens: policy forward/backward on a synthetic rollout, optimizer step; loss and gradient norm
                 finite, weights changed, weights identical on all ranks
  ppo_exercise   (``--ppo-exercise``) one PPO iteration of a few tokens: generate -> reference log-probs -> values ->
                 actor step -> critic step
  checkpoint     (``--checkpoint-dir``) flat-shard save of weights + Adam state, weights scrambled, strict reload,
                 bitwise comparison
  device_status  no bounded device-side wait ran out

Exit code 0 only if every check passed; rank 0 prints the report (``rpeg.engine_validate.v1``).
Reference: RPEG/runtime/megatron_validate.py:57-174 (model build at dp/pp/tp, random-token training step, optional
two-token PPO exercise, distributed checkpoint save + strict reload).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path
from typing import Any, Dict, List, Optional

SCHEMA = "rpeg.engine_validate.v1"


def _entry(name: str, ok: bool, detail: Any, seconds: float) -> Dict[str, Any]:
    return {"name": name, "ok": bool(ok), "detail": detail, "seconds": round(seconds, 3)}


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="engine smoke worker (train step, PPO exercise, checkpoint round trip)")
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--hidden", type=int, default=256)
    ap.add_argument("--ffn", type=int, default=512)
    ap.add_argument("--vocab", type=int, default=512)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--kv-heads", type=int, default=0, help="0 = as many as query heads")
    ap.add_argument("--rows", type=int, default=8, help="sequences per rank in the training step")
    ap.add_argument("--prompt-len", type=int, default=16)
    ap.add_argument("--response-len", type=int, default=16)
    ap.add_argument("--ppo-exercise", action="store_true")
    ap.add_argument("--ppo-tokens", type=int, default=2, help="new tokens per row in the PPO exercise")
    ap.add_argument("--checkpoint-dir", default=None)
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--json", action="store_true", help="print the report as one JSON line")
    return ap


def model_config(args):
    from ..models.llama import LlamaConfig
    if args.hidden % args.head_dim:
        raise SystemExit("--hidden must be a multiple of --head-dim")
    heads = args.hidden // args.head_dim
    return LlamaConfig(n_layers=args.layers, d_model=args.hidden, d_ff=args.ffn, n_heads=heads, n_kv_heads=args.kv_heads or heads,
                       head_dim=args.head_dim, vocab=args.vocab, max_pos=max(512, args.prompt_len + args.response_len + 16))


def validate(args) -> Dict[str, Any]:
    import torch
    import torch.distributed as dist

    from ..engine import algorithms as A
    from ..engine.optimizer import AdamW
    from ..models.llama import LlamaModel
    from ..ops import kernels as K
    from . import checkpoint as ckpt

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    device = torch.device(f"cuda:{int(os.environ.get('LOCAL_RANK', '0'))}")
    torch.cuda.set_device(device)
    dp = None
    if world > 1:
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=device)
        from ..parallel.dp import DPContext
        dp = DPContext(device)
    checks: List[Dict[str, Any]] = []
    cfg = model_config(args)
    algo = A.AlgoConfig(kl_coef=0.0, micro_tokens=max(512, 2 * (args.prompt_len + args.response_len)), head_chunk=min(8192, args.vocab))

    def same_on_all_ranks(t: "torch.Tensor") -> bool:
        if world == 1:
            return True
        s = t.float().sum().double().reshape(1)
        lo, hi = s.clone(), s.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        return bool((lo == hi).item())

    # ---- build
    t0 = time.perf_counter()
    model = LlamaModel(cfg, device, trainable=True, weights=dp.alloc_weights(cfg) if dp else None,
                       grads=dp.alloc_grads(cfg) if dp else None, seed=args.seed)
    model.init_weights(args.seed)
    opt = AdamW(model, lr=1e-3, dp=dp)
    n = model.layout.total
    torch.cuda.synchronize()
    checks.append(_entry("build", True, {"parameters": int(n), "world": world, "device": torch.cuda.get_device_name(device)},
                         time.perf_counter() - t0))

    # ---- train_step: a synthetic rollout (random prompts and responses), ratio 1 against its own log-probs
    t0 = time.perf_counter()
    g = torch.Generator().manual_seed(args.seed + 17 * rank)
    N, S, T = args.rows, args.prompt_len, args.response_len
    prompts = torch.randint(3, cfg.vocab, (N, S), generator=g, dtype=torch.int32).to(device)
    resp = torch.randint(3, cfg.vocab, (N, T), generator=g, dtype=torch.int32).to(device)
    lens = [int(x) for x in torch.randint(max(1, T // 2), T + 1, (N,), generator=g)]
    mask = (torch.arange(T, device=device)[None, :] < torch.tensor(lens, device=device)[:, None]).float()
    ro = A.Rollout(prompts, [S] * N, resp, lens, torch.zeros((N, T), device=device), mask)
    ro.old_logp = A.sequence_logprobs(model, ro, algo)
    ro.adv = torch.randn((N, T), generator=g).to(device) * mask
    before = model.w[:n].float().clone()
    denom = float(ro.n_response_tokens())
    if dp is not None:
        denom = dp.all_reduce_scalar(denom)
    model.zero_grad()
    m = A.policy_train_step(model, ro, algo, denom_tokens=denom)
    opt.step()
    torch.cuda.synchronize()
    loss, gnorm = float(m["loss"]), float(opt.grad_norm())
    moved = float((model.w[:n].float() - before).abs().max())
    ok = loss == loss and abs(loss) < 1e6 and gnorm == gnorm and 0.0 < gnorm < 1e6 and moved > 0.0 and same_on_all_ranks(model.w[:n])
    checks.append(_entry("train_step", ok, {"loss": loss, "grad_norm": gnorm, "max_weight_change": moved, "tokens": int(sum(lens)) + N * S},
                         time.perf_counter() - t0))

    # ---- ppo_exercise
    if args.ppo_exercise:
        t0 = time.perf_counter()
        from ..engine.trainers import PPOTrainer
        tr = PPOTrainer(cfg, device=device, max_new=args.ppo_tokens, prompt_len=S, algo=A.AlgoConfig(micro_tokens=algo.micro_tokens, head_chunk=algo.head_chunk),
                        dp=dp.clone("ppo_actor") if dp else None, gen_slots=max(8, N), kv_budget_bytes=2e9, seed=args.seed, eos_id=1)
        out = tr.step(torch.randint(3, cfg.vocab, (N, S), generator=g, dtype=torch.int32))
        torch.cuda.synchronize()
        vals = {k: float(v) for k, v in out.items() if k in ("loss", "value_loss", "grad_norm", "mean_score", "gen_tokens")}
        checks.append(_entry("ppo_exercise", all(v == v and abs(v) < 1e9 for v in vals.values()) and vals.get("gen_tokens", 1.0) > 0, vals,
                             time.perf_counter() - t0))
        del tr

    # ---- checkpoint round trip
    if args.checkpoint_dir:
        t0 = time.perf_counter()
        d = Path(args.checkpoint_dir) / "engine_validate" / "actor"
        tensors = {"adam.master": opt.master, "adam.m": opt.m, "adam.v": opt.v}
        ranges = {k: (opt.shard_off, opt.shard_off + opt.shard_n, n) for k in tensors}
        if rank == 0:
            tensors["weights"] = model.w[:n]
        ckpt.save_flat_shards(d, rank, world, tensors, ranges=ranges, extra={"optimizer_step": opt.step_count})
        if world > 1:
            dist.barrier()
        if rank == 0:
            ckpt.finalize_worker_meta(d, world, extra={"step": 1, "kind": "validate"})
            ckpt.write_weight_versions(d.parent, step=1, latest={"actor": 1}, retained={"actor": [1]}, tau={"actor": 0})
        if world > 1:
            dist.barrier()
        want_w, want_m = model.w[:n].clone(), opt.m.clone()
        model.w[:n].zero_()
        opt.m.zero_()
        model.w[:n].copy_(ckpt.load_tensor(d, "weights").to(device))
        opt.m.copy_(ckpt.load_flat_range(d, "adam.m", opt.shard_off, opt.shard_off + opt.shard_n).to(device))
        torch.cuda.synchronize()
        same = bool(torch.equal(model.w[:n], want_w)) and bool(torch.equal(opt.m, want_m))
        rep = ckpt.verify_checkpoint(d.parent, ["actor"])
        checks.append(_entry("checkpoint", same and not rep["errors"], {"bitwise_equal": same, "files": rep["files"], "bytes": rep["bytes"],
                                                                       "errors": rep["errors"], "path": str(d)},
                             time.perf_counter() - t0))

    # ---- device status
    try:
        K.check_status()
        checks.append(_entry("device_status", True, "no wait ran out", 0.0))
    except K.KernelWaitTimeout as exc:
        checks.append(_entry("device_status", False, str(exc), 0.0))

    ok = all(c["ok"] for c in checks)
    if world > 1:
        flag = torch.tensor([1.0 if ok else 0.0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        ok = bool(flag.item() == 1.0)
        dist.barrier()
    return {"schema_version": SCHEMA, "ok": ok, "rank": rank, "world": world, "checks": checks,
            "model": {"layers": cfg.n_layers, "hidden_dim": cfg.d_model, "ffn_dim": cfg.d_ff, "vocab_size": cfg.vocab}}


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    try:
        import torch
        if not torch.cuda.is_available():
            print(json.dumps({"schema_version": SCHEMA, "ok": False, "error": "no CUDA device visible"}))
            return 2
    except ImportError as exc:
        print(json.dumps({"schema_version": SCHEMA, "ok": False, "error": str(exc)}))
        return 2
    rep = validate(args)
    if rep["rank"] == 0:
        if args.json:
            print(json.dumps(rep))
        else:
            for c in rep["checks"]:
                print(f"{'ok  ' if c['ok'] else 'FAIL'} {c['name']:<14} {c['seconds']:>8.3f} s  {c['detail']}")
            print("engine validation " + ("passed" if rep["ok"] else "FAILED"))
    elif not rep["ok"]:
        bad = [c for c in rep["checks"] if not c["ok"]]
        if bad:
            print(json.dumps({"rank": rep["rank"], "failed": bad}), file=sys.stderr)
    return 0 if rep["ok"] else 2


if __name__ == "__main__":
    sys.exit(main())
