"""Flagship benchmark: one full RLHF iteration (generation -> reference log-probs -> rewards ->
policy forward/backward -> optimizer) per step, on N GPUs of one node.

    python bench.py --gpus 1 --steps 1 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 2 --warmup 3

Default workload (``--config grpo_7b``): GRPO on random-init Llama-7B-shaped actor + frozen reference,
32 prompts x 8 samples per iteration, 512-token prompts drawn uniformly from the vocabulary (seed 42),
sampled generation up to 2048 tokens with EOS forced at lengths drawn from the quantiles
[0.5 -> 512, 0.9 -> 1024, 1.0 -> 2048], rewards ~ N(0,1) group-normalised, bf16 compute, fp32 Adam.
The total batch is fixed, so more GPUs means strong scaling (data parallel over prompts).

Rank 0 prints ONE JSON line. ``value`` is samples/s over all GPUs from CUDA-event timing of K steps
whose inputs already sit on the device; ``e2e`` repeats K steps through the public ``step`` API with
pinned host inputs (H2D copy) and the loss read back (D2H). ``--impl reference`` reports why the
reference cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

CONFIGS = {
    # name: (model, prompts, samples_per_prompt, prompt_len, max_new, quantiles)
    "grpo_7b": dict(algo="grpo", model="llama7b", prompts=32, k=8, prompt_len=512, max_new=2048,
                    quantiles=((0.5, 512), (0.9, 1024), (1.0, 2048))),
    "grpo_tiny": dict(algo="grpo", model="tiny", prompts=16, k=4, prompt_len=32, max_new=64,
                      quantiles=((0.5, 16), (0.9, 32), (1.0, 64))),
    "dpo_7b": dict(algo="dpo", model="llama7b", prompts=64, k=2, prompt_len=256, max_new=768, quantiles=None),
    # PPO with four 7B-shape models (actor, critic, reference, reward); needs >= 4 GPUs for the two Adam states
    "ppo_7b": dict(algo="ppo", model="llama7b", prompts=64, k=1, prompt_len=128, max_new=512,
                   quantiles=((0.5, 128), (0.85, 256), (1.0, 512)), min_gpus=4),
    # PPO with a shared 13B actor/critic trunk (LM head + value head) and a 7B-shape reward model. Per GPU: 26 GB of bf16
    # weights + 52 GB of fp32 gradients + 156 GB / N of Adam state + the 13.5 GB reward model + the KV pool: 8 GPUs
    # (on 4 the construction runs out of memory at 159 GB in use)
    "ppo_acshare_13b": dict(algo="ppo", model="llama13b", prompts=128, k=1, prompt_len=256, max_new=1024, shared=True,
                            quantiles=((0.5, 256), (0.85, 512), (1.0, 1024)), min_gpus=8),
    "ppo_tiny": dict(algo="ppo", model="tiny", prompts=16, k=1, prompt_len=32, max_new=64, quantiles=((0.5, 16), (0.9, 32), (1.0, 64))),
    "dpo_tiny": dict(algo="dpo", model="tiny", prompts=16, k=2, prompt_len=32, max_new=64, quantiles=None),
    # GRPO with generation and training on disjoint halves of the GPUs and one step of bounded staleness: generation of
    # iteration k + 1 overlaps training of iteration k; weights and rollouts cross through versioned peer-memory channels
    "grpo_7b_async": dict(algo="grpo_async", model="llama7b", prompts=32, k=8, prompt_len=512, max_new=2048, tau=1,
                          quantiles=((0.5, 512), (0.9, 1024), (1.0, 2048)), min_gpus=2),
    # GRPO with data-parallel generation and a pipeline-parallel policy update (1F1B over all ranks, one stage's optimizer
    # state per GPU, weights broadcast back into the replicated generation copy after the step)
    "grpo_7b_pp": dict(algo="grpo", model="llama7b", prompts=32, k=8, prompt_len=512, max_new=2048, pipeline_train=True,
                       quantiles=((0.5, 512), (0.9, 1024), (1.0, 2048)), min_gpus=2),
    "grpo_tiny_pp": dict(algo="grpo", model="tiny", prompts=16, k=4, prompt_len=32, max_new=64, pipeline_train=True,
                         quantiles=((0.5, 16), (0.9, 32), (1.0, 64)), min_gpus=2),
    "grpo_tiny_async": dict(algo="grpo_async", model="tiny", prompts=16, k=4, prompt_len=32, max_new=64, tau=1,
                            quantiles=((0.5, 16), (0.9, 32), (1.0, 64)), min_gpus=2),
}


MODEL_SHAPES = {
    "llama7b": dict(layers=32, hidden=4096, ffn=11008, heads=32, kv_heads=32, vocab=32000),
    "llama13b": dict(layers=40, hidden=5120, ffn=13824, heads=40, kv_heads=40, vocab=32000),
    "tiny": dict(layers=2, hidden=256, ffn=512, heads=2, kv_heads=2, vocab=512),
}
PLANNER_CONFIG = os.path.join(os.path.dirname(os.path.abspath(__file__)), "configs", "example_ppo_32gpu.yaml")


def reference_arm(args, spec, world: int) -> dict:
    """Runs the reference's own code (baseline/ref_arm.py) and returns the JSON line of the reference arm."""
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline"))
    import ref_arm
    from pathlib import Path
    base = {"impl": "reference", "n_gpus": world, "steps": args.steps, "warmup": args.warmup}
    try:
        if args.config == "planner_32gpu":
            r = ref_arm.planner_arm(Path(PLANNER_CONFIG))
            return {**base, "metric": "planner_predicted_tokens_per_sec", "value": r["optimized_tokens_per_s"], "unit": "tokens/s (predicted)",
                    "higher_is_better": True, "search_wall_s": r["search_wall_s"], "detail": r,
                    "config": {"model": "PPO, 3 x 7B-shape, 32 GPUs (1 x 8 x 4), example alpha-beta constants", "seed": 42}}
        if world > 1:
            try:
                import megatron.core  # noqa: F401
                why = "its multi-GPU backend also needs a Slurm launcher, which this box does not have"
            except Exception as exc:  # noqa: BLE001
                why = f"its multi-GPU backend (runtime.default_backend=megatron) needs megatron-core==0.17.0: {type(exc).__name__}: {exc}"
            return {**base, "unavailable": f"reference cannot run on {world} GPUs here: {why}; its torch backend accepts single-device plans only "
                                          "(RPEG/runtime/algorithms/ppo_graph.py:950-963)"}
        import tempfile
        work = Path(tempfile.mkdtemp(prefix="rpeg_ref_arm_"))
        try:
            r = ref_arm.torch_arm(algo=spec["algo"], model=MODEL_SHAPES[spec["model"]], prompts=spec["prompts"], samples_per_prompt=spec["k"],
                                  prompt_len=spec["prompt_len"], max_new=spec["max_new"], quantiles=spec["quantiles"],
                                  steps=max(1, min(args.steps, 3)), warmup=min(args.warmup, 1), workdir=work,
                                  timeout_s=float(args.ref_budget_s))
        finally:
            import shutil
            shutil.rmtree(work, ignore_errors=True)      # the model directory written for the reference is 13.5 GB
        return {**base, "metric": "rlhf_samples_per_sec", "value": r["samples_per_s"], "unit": "samples/s", "higher_is_better": True,
                "steps": r["steps"], "ms_per_step": 1e3 * r["seconds"] / r["steps"], "gen_tokens_per_sec": r["gen_tokens_per_s"],
                "e2e": {"value": r["samples_per_s"], "unit": "samples/s", "note": "the reference's trace is host-timed around each node, input tokenisation and copies included"},
                "dtype": "bf16", "data": "synthetic",
                "config": {"model": f"{spec['model']} (HF LlamaForCausalLM, random init)", "algorithm": spec["algo"], "prompts": spec["prompts"],
                           "samples_per_prompt": spec["k"], "prompt_len": spec["prompt_len"], "max_new_tokens": spec["max_new"],
                           "parallelism": "single device, runtime.default_backend=torch_grpo",
                           "note": "the stock path has no forced EOS lengths: rows stop at EOS or at max_new_tokens"}}
    except ref_arm.ReferenceUnavailable as exc:
        return {**base, "unavailable": str(exc)}
    except Exception as exc:  # noqa: BLE001
        return {**base, "unavailable": f"{type(exc).__name__}: {exc}"}


def planner_bench(args) -> dict:
    """Our planner on the 32-GPU PPO example (CPU only): predicted throughput of the optimized plan and search wall time."""
    import contextlib
    import io
    import re
    from rpeg_b200.planner import pipeline as planner
    buf = io.StringIO()
    t0 = time.perf_counter()
    with contextlib.redirect_stdout(buf):
        planner.main(["--config", PLANNER_CONFIG])
    wall = time.perf_counter() - t0
    out = buf.getvalue()
    m = re.search(r"Throughput \(tokens/s\)\s+(\S+)\s+(\S+)\s+(\S+)", out)
    mw = re.search(r"wall time\s+([0-9.]+)\s*s", out)
    if not m:
        raise SystemExit("planner printed no result table:\n" + out[-2000:])
    return {"impl": "ours", "metric": "planner_predicted_tokens_per_sec", "value": float(m.group(3)), "unit": "tokens/s (predicted)",
            "higher_is_better": True, "n_gpus": 0, "steps": 1, "warmup": 0, "search_wall_s": float(mw.group(1)) if mw else wall,
            "process_wall_s": wall, "greedy_tokens_per_s": float(m.group(1)), "heuristic_tokens_per_s": float(m.group(2)),
            "gpu_launches": 0, "data": "synthetic",
            "config": {"model": "PPO, 3 x 7B-shape, 32 GPUs (1 x 8 x 4), example alpha-beta constants", "seed": 42}}


class ClockSampler:
    """Samples SM clocks / throttle reasons of the job's GPUs with ONE nvidia-smi process while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, indices):
        self.indices = [int(i) for i in (indices if isinstance(indices, (list, tuple, range)) else [indices])]
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "250", "-i", ",".join(str(i) for i in self.indices)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        per_gpu, mx, reasons = {}, [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 8:
                continue
            try:
                per_gpu.setdefault(int(parts[0]), []).append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm = sorted(v for vals in per_gpu.values() for v in vals)
        out = {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
               "reasons": sorted(reasons), "samples": len(sm)}
        if len(per_gpu) > 1:      # the slowest GPU sets the pace of a step: show every GPU's median
            out["sm_mhz_per_gpu"] = {str(g): sorted(v)[len(v) // 2] for g, v in sorted(per_gpu.items())}
        return out


def draw_lengths(n: int, quantiles, gen) -> "list[int]":
    """Per-row generation length: a row finishes in bucket q with the bucket's probability mass and
    is cut uniformly inside (previous bound, bound]."""
    import torch
    u = torch.rand(n, generator=gen)
    lo, out = 0, torch.zeros(n, dtype=torch.long)
    prev = 0.0
    for frac, bound in quantiles:
        sel = (u >= prev) & (u < frac) if frac < 1.0 else (u >= prev)
        width = bound - lo
        out[sel] = lo + 1 + (torch.rand(int(sel.sum()), generator=gen) * width).long().clamp(max=width - 1)
        prev, lo = frac, bound
    return out.tolist()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="grpo_7b", choices=sorted(CONFIGS) + ["planner_32gpu"])
    ap.add_argument("--gen-slots", type=int, default=0)
    ap.add_argument("--kv-gb", type=float, default=0.0, help="KV cache budget per GPU in GB (0 = pick by world size)")
    ap.add_argument("--micro-tokens", type=int, default=16384)
    ap.add_argument("--gen-tp-size", type=int, default=0, help="tensor-parallel generation in groups of this many consecutive ranks "
                    "(a divisor of --gpus; generation layout (gpus / t, 1, t)); 0 = one group of all ranks")
    ap.add_argument("--recompute", default="auto", choices=["auto", "full", "none"])
    ap.add_argument("--ref-budget-s", type=float, default=480.0, help="--impl reference: seconds the reference's own run may take "
                    "(writing its model directory included) before the arm reports it as unavailable")
    ap.add_argument("--gen-parallel", default="auto", choices=["auto", "dp", "tp"],
                    help="generation layout on more than one GPU: tensor parallel over all ranks (every rank decodes the whole "
                         "batch on its weight shard) or data parallel (every rank decodes its rows on the whole model); auto = tp")
    ap.add_argument("--tp-comm", default=None, choices=["auto", "nvls", "peer"],
                    help="tensor-parallel decode collectives: NVLS multimem or plain peer loads/stores (default: RPEG_TP_COMM or auto)")
    ap.add_argument("--group-attention", default="off", choices=["off", "cuda", "tc"],
                    help="GRPO: score the K samples of a prompt against the prompt's shared KV pages once per group (CUDA-core or "
                         "tcgen05 kernel) instead of once per row through L2; off by default: measured slower on the full step")
    ap.add_argument("--budget-s", type=float, default=420.0,
                    help="wall-clock budget for warm-up plus timed steps; the timed step count is cut to fit and reported")
    args = ap.parse_args()
    # Libraries (NCCL's version banner, for one) write to file descriptor 1. The contract is ONE JSON line on
    # stdout, so everything else is sent to stderr and the line goes to the saved descriptor at the end.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)

    def emit(obj) -> None:
        sys.stdout.flush()
        os.write(real_stdout, (json.dumps(obj) + "\n").encode())

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        if rank == 0:
            emit(reference_arm(args, CONFIGS.get(args.config), world))
        return
    if args.config == "planner_32gpu":
        if rank == 0:
            emit(planner_bench(args))
        return
    if world != args.gpus:
        if args.gpus == 1 and world == 1:
            pass
        else:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")

    import torch
    import torch.distributed as dist

    from rpeg_b200.engine import algorithms as A
    from rpeg_b200.engine.trainers import DPOTrainer, GRPOTrainer
    from rpeg_b200.models.llama import LlamaConfig
    from rpeg_b200.ops import _lib
    from rpeg_b200.ops import kernels as K

    torch.cuda.set_device(local_rank)
    device = torch.device(f"cuda:{local_rank}")
    spec = CONFIGS[args.config]
    dp = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
        if spec["algo"] != "grpo_async" and not spec.get("pipeline_train"):   # those engines build their own groups
            from rpeg_b200.parallel.dp import DPContext
            dp = DPContext(device)

    if world < spec.get("min_gpus", 1):
        raise SystemExit(f"config {args.config} needs at least {spec['min_gpus']} GPUs (optimizer state of its trainable models)")
    cfg = {"llama7b": lambda: LlamaConfig.llama7b(max_pos=4096), "llama13b": lambda: LlamaConfig.llama13b(max_pos=4096),
           "tiny": LlamaConfig.tiny}[spec["model"]]()
    B, Kk, S, T = spec["prompts"], spec["k"], spec["prompt_len"], spec["max_new"]
    if B % world and spec["algo"] != "grpo_async":
        raise SystemExit(f"{B} prompts do not split over {world} ranks")
    b_local = B // world
    recompute = args.recompute
    if recompute == "auto":
        recompute = "full"
    algo = A.AlgoConfig(kl_coef=0.04, beta=0.1, micro_tokens=args.micro_tokens, head_chunk=8192)

    gen_host = torch.Generator().manual_seed(42)
    n_iters = min(args.warmup + args.steps, 12)   # distinct synthetic batches; the loop cycles through them
    if spec["algo"] == "grpo":
        # KV pages are handed out on demand, so the slot count may exceed what the budget holds at full length.
        # One rank keeps the whole fp32 Adam state (81 GB for 7B) and has ~56 GB for KV; sharded ranks have more.
        # the K samples of a prompt share its KV pages, so the pool holds every row of the rank at once
        gen_tp = world > 1 and args.gen_parallel in ("auto", "tp") and not spec.get("pipeline_train")
        tp_size = (args.gen_tp_size or world) if gen_tp else 1
        if gen_tp and (tp_size < 2 or world % tp_size):
            raise SystemExit(f"--gen-tp-size {tp_size} must be a divisor (>= 2) of the {world} GPUs")
        slots = args.gen_slots or min((B * tp_size // world if gen_tp else b_local) * Kk, 256)
        # tensor-parallel generation: a rank holds 1/t of the heads of every row of its group, so the token capacity that
        # one GPU gets from 56 GB needs 56 / t GB per rank (half as much again is kept as head room)
        kv_gb = args.kv_gb or ((84.0 / tp_size) if gen_tp else {1: 56.0, 2: 76.0}.get(world, 96.0))
        if spec.get("pipeline_train"):
            from rpeg_b200.engine.trainers import PipelineGRPOTrainer
            trainer = PipelineGRPOTrainer(cfg, device=device, samples_per_prompt=Kk, max_new=T, prompt_len=S, algo=algo,
                                          gen_slots=slots, kv_budget_bytes=kv_gb * 1e9, recompute=recompute, seed=42, eos_id=2)
        else:
            def build(tp: bool, slots_: int, kv_gb_: float, dp_):
                return GRPOTrainer(cfg, device=device, samples_per_prompt=Kk, max_new=T, prompt_len=S, algo=algo, dp=dp_,
                                   gen_slots=slots_, kv_budget_bytes=kv_gb_ * 1e9, recompute=recompute, seed=42, eos_id=2,
                                   gen_tp=tp, tp_comm=args.tp_comm, gen_tp_size=(tp_size if tp and tp_size != world else None),
                                   group_attention={"off": False, "cuda": True, "tc": "tc"}[args.group_attention])

            trainer = build(gen_tp, slots, kv_gb, dp)
            if gen_tp and args.gen_parallel == "auto":
                # Before a long run: the tensor-parallel decode step against the whole local model on a few rows (both
                # all-reduce kernels). If any rank disagrees, or a peer does not answer within the kernels' bounded waits,
                # all ranks fall back to data-parallel generation instead of failing the job.
                why = None
                try:
                    err = trainer.gen_model.selfcheck(rows=(8, max(64, 512 // world)))
                    if not (err < 5e-2) or os.environ.get("RPEG_BENCH_FORCE_TP_FALLBACK") == "1":
                        why = f"decode step differs from the whole model by {err:.3g}"
                except Exception as exc:  # noqa: BLE001
                    why = f"{type(exc).__name__}: {exc}"
                    K.status_word(device).zero_()
                bad = torch.tensor([0 if why is None else 1], device=device)
                dist.all_reduce(bad, op=dist.ReduceOp.MAX)
                if int(bad.item()):
                    if rank == 0:
                        print(f"[bench] tensor-parallel generation failed its start-up check ({why or 'on another rank'}): "
                              "generating data parallel", file=sys.stderr, flush=True)
                    trainer.gen_model.comm.close()
                    del trainer
                    import gc
                    gc.collect()
                    torch.cuda.empty_cache()
                    from rpeg_b200.parallel.dp import DPContext
                    gen_tp = False
                    slots = args.gen_slots or min(b_local * Kk, 256)
                    kv_gb = args.kv_gb or {1: 56.0, 2: 76.0}.get(world, 96.0)
                    dp = DPContext(device, tag="actor2")
                    trainer = build(False, slots, kv_gb, dp)
                else:
                    torch.cuda.empty_cache()          # the check's scratch KV caches go back to the driver
                    if rank == 0:
                        print(f"[bench] tensor-parallel start-up check: max relative difference {err:.3g}", file=sys.stderr, flush=True)
        batches = []
        for _ in range(n_iters):
            prompts = torch.randint(3, cfg.vocab, (B, S), generator=gen_host, dtype=torch.int32)
            rewards = torch.randn(B * Kk, generator=gen_host)
            lens = torch.tensor(draw_lengths(B * Kk, spec["quantiles"], gen_host), dtype=torch.int32)
            sl_p, sl_r = slice(rank * b_local, (rank + 1) * b_local), slice(rank * b_local * Kk, (rank + 1) * b_local * Kk)
            batches.append((prompts[sl_p].contiguous().pin_memory(), rewards[sl_r].contiguous().pin_memory(), lens[sl_r].contiguous()))

        def run(i, on_device):
            p, r, l = batches[i]
            if on_device:
                p, r = p.to(device), r.to(device)
            return trainer.step(p, r, forced_lens=l)
    elif spec["algo"] == "grpo_async":
        import types
        from rpeg_b200.engine.async_rl import AsyncGRPO
        half = world // 2
        n_gen_rows = B * Kk // half
        slots = args.gen_slots or min(n_gen_rows, 256)
        eng = AsyncGRPO(cfg, gen_ranks=list(range(half)), train_ranks=list(range(half, world)), prompts_per_step=B,
                        samples_per_prompt=Kk, max_new=T, prompt_len=S, tau=int(spec.get("tau", 1)), algo=algo, gen_slots=slots,
                        kv_budget_bytes=(args.kv_gb or 96.0) * 1e9, seed=42, eos_id=2, device=device, wait_timeout_s=900.0)
        trainer = types.SimpleNamespace(h2d_bytes=0, d2h_bytes=0, last_counters={})
        batches = []
        for _ in range(n_iters):
            prompts = torch.randint(3, cfg.vocab, (B, S), generator=gen_host, dtype=torch.int32)
            rewards = torch.randn(B * Kk, generator=gen_host)
            lens = draw_lengths(B * Kk, spec["quantiles"], gen_host)
            batches.append((prompts.pin_memory(), rewards.pin_memory(), lens))

        def run(i, on_device):
            p, r, l = batches[i]
            trainer.h2d_bytes = p.numel() * p.element_size() + (r.numel() * r.element_size() if eng.is_train else 0)
            trainer.d2h_bytes = 8
            if on_device:
                p, r = p.to(device), r.to(device)
            out = eng.step(p, r, forced_lens=l)
            trainer.last_counters = dict(eng.counters)
            out.setdefault("samples", 0.0)
            out.setdefault("gen_tokens", 0.0)
            out.setdefault("train_tokens", 0.0)
            return out
    elif spec["algo"] == "ppo":
        from rpeg_b200.engine.trainers import PPOTrainer
        slots = args.gen_slots or min(b_local * Kk, 128)
        reward_cfg = LlamaConfig.llama7b(max_pos=4096) if spec["model"] == "llama13b" else None
        trainer = PPOTrainer(cfg, device=device, max_new=T, prompt_len=S, algo=algo, dp=dp, gen_slots=slots,
                             kv_budget_bytes=(args.kv_gb or 40.0) * 1e9, recompute=recompute, seed=42, eos_id=2,
                             share_actor_critic=bool(spec.get("shared", False)), reward_cfg=reward_cfg)
        batches = []
        for _ in range(n_iters):
            prompts = torch.randint(3, cfg.vocab, (B, S), generator=gen_host, dtype=torch.int32)
            lens = torch.tensor(draw_lengths(B, spec["quantiles"], gen_host), dtype=torch.int32)
            sl = slice(rank * b_local, (rank + 1) * b_local)
            batches.append((prompts[sl].contiguous().pin_memory(), lens[sl].contiguous()))

        def run(i, on_device):
            p, l = batches[i]
            if on_device:
                p = p.to(device)
            return trainer.step(p, forced_lens=l)
    else:
        trainer = DPOTrainer(cfg, device=device, algo=algo, dp=dp, recompute=recompute, seed=42)
        batches = []
        for _ in range(n_iters):
            pr = torch.randint(3, cfg.vocab, (B, S), generator=gen_host, dtype=torch.int32).repeat_interleave(2, 0)
            rs = torch.randint(3, cfg.vocab, (2 * B, T), generator=gen_host, dtype=torch.int32)
            sl = slice(rank * 2 * b_local, (rank + 1) * 2 * b_local)
            batches.append((pr[sl].contiguous().pin_memory(), rs[sl].contiguous().pin_memory()))

        def run(i, on_device):
            p, r = batches[i]
            if on_device:
                p, r = p.to(device), r.to(device)
            return trainer.step(p, r)

    # Recomputation policy. "auto": keep the activations of as many layers for the backward pass as this rank has the
    # memory for (their second forward pass is skipped: up to a quarter fewer training FLOPs) and recompute the other
    # layers from their inputs. One layer's activations of a microbatch are micro_tokens x (7 d + 3 d_ff) bf16 values plus
    # the attention statistics. If not all layers fit with the requested microbatch and more fit with half of it, it is halved
    # (same tokens per step, twice the launches). All ranks take the smallest answer.
    keep_layers = None
    if args.recompute == "auto":
        policy = None
        for name in ("actor", "policy"):
            if hasattr(trainer, name):
                policy = getattr(trainer, name)
        if policy is not None and getattr(policy, "g", None) is not None:
            torch.cuda.synchronize()
            free_bytes = float(torch.cuda.mem_get_info(device)[0])
            n_l = cfg.n_layers

            from rpeg_b200.engine.memory_policy import choose_kept_layers, layers_that_fit as _fit

            def layers_that_fit(micro: int) -> int:
                return _fit(free_bytes, n_l, cfg.d_model, cfg.d_ff, micro)

            fit, micro = choose_kept_layers(free_bytes, n_l, cfg.d_model, cfg.d_ff, args.micro_tokens)
            choice = torch.tensor([fit, micro], device=device, dtype=torch.int64)
            if world > 1:
                dist.all_reduce(choice, op=dist.ReduceOp.MIN)
            keep_layers, micro = int(choice[0].item()), int(choice[1].item())
            if micro != args.micro_tokens:
                keep_layers = min(keep_layers, layers_that_fit(micro))
                args.micro_tokens = micro
                algo.micro_tokens = micro
            recompute = "none" if keep_layers == n_l else ("full" if keep_layers == 0 else f"all but the last {keep_layers} layers")
            for name in ("actor", "policy", "critic"):
                m_ = getattr(trainer, name, None)
                if m_ is not None and getattr(m_, "g", None) is not None:
                    m_.recompute = "none" if keep_layers == n_l else "full"
                    m_.keep_layers = 0 if keep_layers == n_l else keep_layers
            if rank == 0:
                print(f"[bench] recompute={recompute}: {free_bytes / 1e9:.1f} GB free, microbatch of {micro} tokens, "
                      f"activations of one layer {1.15 * micro * (7 * cfg.d_model + 3 * cfg.d_ff) * 2 / 1e9:.2f} GB",
                      file=sys.stderr, flush=True)
    recompute_state = {"value": recompute}
    parallelism_text = getattr(trainer, "parallelism", None) or f"dp{world}"

    def extra_metrics(line: dict) -> dict:
        """The two remaining headline quantities: device time of the weight hand-over from the training layout to the
        generation layout per iteration, and the planner's predicted step time against the measured one."""
        extra = {}
        reshard = getattr(trainer, "last_reshard_us", None)
        if reshard is not None:
            extra["reshard_us"] = float(reshard)
        try:
            from rpeg_b200.analytic.predict import predict_step_seconds
            frac = 0.0 if recompute == "none" else (1.0 if not keep_layers else max(0.0, 1.0 - keep_layers / cfg.n_layers))
            pred = predict_step_seconds(spec, world, parallelism=line["config"]["parallelism"], recompute_fraction=frac)
            meas = line["ms_per_step"] / 1e3
            extra["cost_model"] = {"predicted_s": pred["step_s"], "measured_s": meas, "err": (pred["step_s"] - meas) / meas,
                                   "phases_s": pred.get("phases_s"), "hardware": pred.get("hardware")}
            extra["cost_model_err"] = abs(pred["step_s"] - meas) / meas
            if world >= 4 and spec["algo"] == "grpo" and not spec.get("pipeline_train"):
                # what the model expects from the other generation layouts on this many GPUs (--gen-tp-size)
                try:
                    alts = {}
                    for t in [t for t in range(2, world + 1) if world % t == 0 and cfg.n_heads % t == 0]:
                        name = f"tp{t}" if t == world else f"dp{world // t} x tp{t}"
                        alts[name] = round(predict_step_seconds(spec, world, parallelism=f"generation {name}",
                                                                recompute_fraction=frac)["step_s"], 3)
                    alts[f"dp{world}"] = round(predict_step_seconds(spec, world, parallelism=f"dp{world}", recompute_fraction=frac)["step_s"], 3)
                    extra["cost_model"]["predicted_s_by_generation_layout"] = alts
                except Exception:  # noqa: BLE001 - an extra, never at the cost of the prediction above
                    pass
        except Exception as exc:  # noqa: BLE001 - the prediction is a report, it must not fail the measurement
            extra["cost_model"] = {"unavailable": f"{type(exc).__name__}: {exc}"}
        return extra

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def fail(where: str, exc: BaseException) -> None:
        """A failed step ends the run at once: the line carries the error, the exit code is non-zero."""
        emit({"metric": "rlhf_samples_per_sec", "value": None, "impl": "ours", "n_gpus": world, "rank": rank,
              "error": f"{where}: {type(exc).__name__}: {exc}"})
        sys.stderr.flush()
        if world > 1:
            # The peers find out through their own bounded waits (5 s). Leave only after they had time to stop
            # launching kernels that address this rank's memory.
            time.sleep(9.0)
        os._exit(1)

    def checked_run(i: int, tag: str):
        """One iteration through the public API (pinned host inputs in, python floats out), then the device status
        word: a kernel whose bounded wait ran out must not let later steps run on its output."""
        t = time.perf_counter()
        try:
            try:
                out = run(i % len(batches), on_device=False)
            except torch.cuda.OutOfMemoryError:
                # kept activations did not fit after all (allocator fragmentation): on one GPU nothing else is in flight,
                # so fall back to recomputing every layer and run the step again; with peers the step cannot be re-entered
                if world > 1 or tag != "warmup" or not keep_layers:
                    raise
                for name in ("actor", "policy", "critic"):
                    m_ = getattr(trainer, name, None)
                    if m_ is not None and getattr(m_, "g", None) is not None:
                        m_.recompute, m_.keep_layers = "full", 0
                        m_.g.zero_()
                recompute_state["value"] = "full (kept activations ran out of memory)"
                torch.cuda.empty_cache()
                print("[bench] out of memory with kept activations: recomputing every layer", file=sys.stderr, flush=True)
                out = run(i % len(batches), on_device=False)
            K.check_status()
        except BaseException as exc:  # noqa: BLE001 - reported and re-raised as the exit code
            fail(f"{tag} step {i}", exc)
        if rank == 0:
            print(f"[bench] {tag} {i}: {time.perf_counter() - t:.2f} s  " +
                  " ".join(f"{k}={v:.0f}" for k, v in out.items() if k.endswith("_ms")), file=sys.stderr, flush=True)
        return out

    def agree(value: float) -> float:
        """The same number on every rank (the slowest rank's), so all ranks take the same decisions."""
        if world == 1:
            return value
        t = torch.tensor([value], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # Warm-up: at least three steps (graph capture, allocator growth, clocks), more only while they are cheap.
    t_begin = time.perf_counter()
    budget = float(args.budget_s)
    n_warm = 0
    step_s = 0.0
    while n_warm < max(args.warmup, 0):
        t = time.perf_counter()
        checked_run(n_warm, "warmup")
        step_s = agree(time.perf_counter() - t)
        n_warm += 1
        spent = agree(time.perf_counter() - t_begin)
        if n_warm >= min(3, args.warmup) and spent + step_s * 2 > 0.35 * budget:
            break
    spent = agree(time.perf_counter() - t_begin)
    n_steps = args.steps
    if step_s > 0.0:
        n_steps = max(1, min(args.steps, int((budget - spent) / (1.08 * step_s))))

    sampler = ClockSampler(list(range(world)) if world > 1 else local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    launches0 = _lib.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    ev0.record()
    outs = [checked_run(n_warm + j, "timed") for j in range(n_steps)]
    ev1.record()
    barrier()
    wall = time.perf_counter() - t0
    launches = _lib.launch_count() - launches0
    clocks = None
    if rank == 0:
        try:
            clocks = sampler.stop()
        except Exception as exc:  # noqa: BLE001 - a malformed sampler line must not cost the measurement
            clocks = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [f"clock sampler failed: {type(exc).__name__}: {exc}"]}
    # e2e: CUDA events around the K public-API calls (pinned-host inputs copied in, metrics read back, every step).
    # value: the same K steps without the copies - per step, the events the trainer records after its inputs are on
    # the device and after its last optimizer kernel. Both are the maximum over ranks.
    dev_ms = sum(o.get("device_ms", 0.0) for o in outs)
    times = torch.tensor([ev0.elapsed_time(ev1), dev_ms if dev_ms > 0.0 else ev0.elapsed_time(ev1)], device=device, dtype=torch.float64)
    stats = torch.tensor([sum(o["samples"] for o in outs), sum(o.get("gen_tokens", 0.0) for o in outs),
                          sum(o["train_tokens"] for o in outs)], device=device, dtype=torch.float64)
    phase_keys = sorted({k for o in outs for k in o if k.endswith("_ms") and k != "device_ms"})
    phases = torch.tensor([sum(o.get(k, 0.0) for o in outs) / n_steps for k in phase_keys], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(stats)
        if len(phase_keys):
            dist.all_reduce(phases, op=dist.ReduceOp.MAX)
    ms_e2e, ms = times.tolist()
    stats = stats.tolist()

    if rank == 0:
        secs = ms / 1e3
        algo_name = spec["algo"]
        model_txt = {"grpo": f"{spec['model']} x2 (actor + frozen reference)", "grpo_async": f"{spec['model']} x2 (actor + frozen reference)",
                     "dpo": f"{spec['model']} x2 (policy + frozen reference)",
                     "ppo": f"{spec['model']} actor" + ("+critic shared trunk" if spec.get("shared") else ", critic") + ", reference, reward"}[algo_name]
        if algo_name == "grpo_async":
            par = f"gen{world // 2}+train{world - world // 2}, staleness {spec.get('tau', 1)}"
        elif spec.get("pipeline_train"):
            par = f"generation dp{world}, training pp{world}"
        else:
            par = parallelism_text
        phase_ms = {k: round(v, 3) for k, v in zip(phase_keys, phases.tolist())}
        line = {
            "metric": "rlhf_samples_per_sec", "value": stats[0] / secs, "unit": "samples/s", "n_gpus": world,
            "steps": n_steps, "warmup": n_warm, "steps_requested": args.steps, "warmup_requested": args.warmup,
            "ms_per_step": ms / n_steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
            "gen_tokens_per_sec": stats[1] / secs, "train_tokens_per_sec": stats[2] / secs,
            "config": {"model": model_txt + ", random init", "algorithm": algo_name,
                       "global_batch": B * Kk if algo_name in ("grpo", "grpo_async") else B, "prompts": B, "samples_per_prompt": Kk,
                       "seq_len": S + T, "prompt_len": S, "max_new_tokens": T, "gen_quantiles": spec["quantiles"],
                       "parallelism": par, "optimizer": "adamw fp32 master, sharded over dp",
                       "recompute": recompute_state["value"], "micro_tokens": args.micro_tokens, "gen_slots": slots if algo_name in ("grpo", "grpo_async", "ppo") else None,
                       "l2": "working set (13.5 GB of weights per model) far exceeds the 126 MB L2; no flush needed",
                       "time_budget_s": budget},
            "e2e": {"value": stats[0] / (ms_e2e / 1e3), "unit": "samples/s", "ms_per_step": ms_e2e / n_steps,
                    "wall_s_per_step": wall / n_steps, "h2d_bytes_per_step": int(trainer.h2d_bytes),
                    "d2h_bytes_per_step": int(trainer.d2h_bytes), "gen_tokens_per_sec": stats[1] / (ms_e2e / 1e3)},
            "timing": "one loop of public-API steps; e2e = CUDA events around the loop (pinned H2D + metric D2H every step); "
                      "value = sum of the per-step device intervals (inputs on device -> last optimizer kernel); max over ranks",
            "gpu_launches": int(launches), "clocks": clocks,
            "phase_ms_per_step": phase_ms,
            "last_step": {k: round(v, 6) for k, v in outs[-1].items()},
            "generation_counters": dict(getattr(trainer, "last_counters", {}) or {}),
            "published_other_hw": "reference paper data: 7B PPO on 8xA100-40GB, 1.73 samples/s (different config)",
        }
        line.update(extra_metrics(line))
        emit(line)
    if world > 1:
        gm = getattr(trainer, "gen_model", None)
        if getattr(gm, "comm", None) is not None:
            gm.comm.close()                      # no kernel addresses a peer after this barrier
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
