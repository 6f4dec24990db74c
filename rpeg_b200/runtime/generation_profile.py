"""Response-length profile: measured completion lengths -> the cumulative quantiles that split the
generation vertex into phases (``workload.gen_quantiles``).

    python -m rpeg_b200.runtime.generation_profile --lengths lengths.json --max-new-tokens 2048 --output profile.json
    python -m rpeg_b200.runtime.generation_profile --sample --config run.yaml --prompts 64 --output profile.json

``--lengths`` reads a JSON list of observed completion lengths (e.g. from an earlier run's trace);
``--sample`` generates with the run file's actor on this GPU and records the lengths. The output
(``rpeg.generation_profile.v1``) holds ``quantiles`` as ``[fraction, tokens]`` pairs at the requested
fractions, rounded up to a multiple of the KV page so a phase boundary never splits a page, the last
one pinned to ``max_new_tokens``. ``runtime.job_plan`` ingests it through ``generation_profile.path``.
Reference: RPEG/runtime/generation_profile.py:24-160.
"""
from __future__ import annotations

import argparse
import json
import math
import sys
from typing import List, Optional, Sequence

SCHEMA = "rpeg.generation_profile.v1"


def quantiles_from_lengths(lengths: Sequence[int], max_new_tokens: int, fractions: Sequence[float] = (0.5, 0.9, 1.0),
                           round_to: int = 64) -> List[List[float]]:
    if not lengths:
        raise ValueError("no lengths to profile")
    xs = sorted(min(int(l), max_new_tokens) for l in lengths)
    out: List[List[float]] = []
    prev_t = 0
    for f in fractions:
        if not 0 < f <= 1:
            raise ValueError("fractions must be in (0, 1]")
        idx = min(len(xs) - 1, max(0, math.ceil(f * len(xs)) - 1))
        t = max_new_tokens if f >= 1.0 else min(max_new_tokens, -(-xs[idx] // round_to) * round_to)
        if t <= prev_t:                   # boundaries must strictly increase: merge degenerate phases
            continue
        out.append([float(f), int(t)])
        prev_t = t
    if not out or out[-1][1] != max_new_tokens or out[-1][0] != 1.0:
        out = [q for q in out if q[1] < max_new_tokens and q[0] < 1.0] + [[1.0, int(max_new_tokens)]]
    return out


def build_profile(lengths: Sequence[int], max_new_tokens: int, fractions=(0.5, 0.9, 1.0), source: str = "lengths") -> dict:
    xs = [int(l) for l in lengths]
    return {"schema_version": SCHEMA, "source": source, "samples": len(xs), "max_new_tokens": int(max_new_tokens),
            "mean_length": sum(xs) / len(xs), "max_length": max(xs), "truncated_fraction": sum(1 for l in xs if l >= max_new_tokens) / len(xs),
            "quantiles": quantiles_from_lengths(xs, max_new_tokens, fractions)}


def sample_lengths(config_path: str, n_prompts: int) -> List[int]:
    import torch
    from ..engine.generation import Generator
    from ..models.llama import LlamaModel
    from .engine_backend import llama_config_from_run
    from .schema import RuntimeRunConfig
    run = RuntimeRunConfig.load(config_path)
    w = run.workload
    dev = torch.device("cuda:0")
    model = LlamaModel(llama_config_from_run(run.models["actor"], w.context_length + w.generation_length), dev, seed=run.algorithm.seed)
    gen = Generator(model, max_slots=min(64, n_prompts), max_seq_len=w.context_length + w.generation_length, kv_budget_bytes=8e9,
                    eos_id=run.tokenizer.eos_token_id)
    g = torch.Generator().manual_seed(run.data.data_seed)
    prompts = torch.randint(3, run.models["actor"].vocab_size, (n_prompts, w.context_length), generator=g, dtype=torch.int32).to(dev)
    res = gen.generate(prompts, w.generation_length, temperature=run.algorithm.temperature, seed=run.algorithm.seed)
    return [int(x) for x in res.lengths.tolist()]


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="Completion-length profile -> generation quantiles")
    ap.add_argument("--lengths", default=None, help="JSON list of completion lengths")
    ap.add_argument("--sample", action="store_true")
    ap.add_argument("--config", default=None)
    ap.add_argument("--prompts", type=int, default=64)
    ap.add_argument("--max-new-tokens", type=int, default=None)
    ap.add_argument("--fractions", default="0.5,0.9,1.0")
    ap.add_argument("--output", required=True)
    args = ap.parse_args(argv)
    fr = tuple(float(x) for x in args.fractions.split(","))
    if args.sample:
        if not args.config:
            ap.error("--sample needs --config")
        from .schema import RuntimeRunConfig
        lengths, source = sample_lengths(args.config, args.prompts), "sampled"
        max_new = args.max_new_tokens or RuntimeRunConfig.load(args.config).workload.generation_length
    else:
        if not args.lengths or not args.max_new_tokens:
            ap.error("--lengths needs --max-new-tokens")
        lengths, source, max_new = json.load(open(args.lengths)), "lengths", args.max_new_tokens
    prof = build_profile(lengths, max_new, fr, source)
    with open(args.output, "w") as f:
        json.dump(prof, f, indent=2)
    print(json.dumps({k: v for k, v in prof.items()}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
