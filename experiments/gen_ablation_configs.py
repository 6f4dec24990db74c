"""Write the search-ablation configurations: three scenarios x ten variants x five seeds.

    python experiments/gen_ablation_configs.py [--out configs/ablation] [--scenarios deep,tight,wide]

Scenarios (PPO, all on B200 nodes of 8 GPUs):
  deep    64 GPUs, 7B actor with 70B critic and reward, B=512, T=128: deep pipelines pay off
  tight   16 GPUs, three 13B models, B=256, T=384: memory is the binding constraint
  wide    32 GPUs, three 7B models, B=512, T=896: long generation, many equally good placements
Variants: baseline; A1 no generation/inference overlap (no length quantiles); A2 synchronous only;
A3 fixed microbatch counts; A4 no pair moves; A5 no warm restarts; A6 uniform vertex choice;
A7 no polish; A8 hard rejection of memory-infeasible plans; A9 geometric cooling.
Each file differs from its scenario's baseline only by the ablated knob and the seed.
Same variants as the reference's experiments/gen_ablation_{deep,tight,wide}.py (ABLATIONS list :161-172).
"""
from __future__ import annotations

import argparse
import copy
import sys
from pathlib import Path

import yaml

sys.path.insert(0, str(Path(__file__).resolve().parent))
from gen_scaling_configs import hardware_section, model, quantiles  # noqa: E402

SEEDS = (1, 2, 3, 4, 5)
SCENARIOS = {
    "deep": dict(gpus=64, actor="7b", critic="70b", reward="70b", B=512, T=128, budget=30000),
    "tight": dict(gpus=16, actor="13b", critic="13b", reward="13b", B=256, T=384, budget=45000),
    "wide": dict(gpus=32, actor="7b", critic="7b", reward="7b", B=512, T=896, budget=40000),
}


def _set(section: str, **kv):
    def apply(cfg: dict) -> None:
        cfg[section].update(kv)
    return apply


def _drop_quantiles(cfg: dict) -> None:
    cfg["workload"].pop("gen_quantiles", None)


ABLATIONS = (
    ("baseline", lambda cfg: None),
    ("A1_no_gen_inf_overlap", _drop_quantiles),
    ("A2_sync_only", _set("optimizer", staleness_candidates={"actor": [0], "critic": [0]})),
    ("A3_fixed_mb", _set("optimizer", fixed_mb=True)),
    ("A4_no_pair_moves", _set("optimizer", alpha_pair=0.0)),
    ("A5_no_restarts", _set("optimizer", stag_window=999999)),
    ("A6_uniform_vertex", _set("optimizer", uniform_vertex=True)),
    ("A7_no_polish", _set("optimizer", no_polish=True)),
    ("A8_hard_oom", _set("optimizer", hard_oom=True)),
    ("A9_geometric_cooling", _set("optimizer", t_init=0.30, t_warm=0.10, t_min=0.01, geometric_cooling=True)),
)


def base_config(name: str) -> dict:
    s = SCENARIOS[name]
    return {
        "hardware": hardware_section(s["gpus"], 8, "b200"),
        "models": {"actor": model(s["actor"]), "critic": model(s["critic"]), "reward": model(s["reward"])},
        "workload": {"batch_size": s["B"], "samples_per_prompt": 1, "context_length": 128, "generation_length": s["T"],
                     "gen_quantiles": quantiles(s["T"])},
        "policy": {"algorithm": "ppo", "allow_ac_share": False},
        "optimizer": {"k_eval": 8, "e_max": s["budget"], "e_struct": s["budget"], "k_x": 6, "t_max": 50, "t_init": 0.05, "t_warm": 0.10,
                      "t_min": 0.05, "stag_window": 10, "lambda_ac": 0.0, "score_eps": 1e-4,
                      "staleness_candidates": {"actor": [0, 1], "critic": [0]}},
        "output": {"plots": False},
    }


def generate(out_dir, scenarios=tuple(SCENARIOS)) -> int:
    out_dir = Path(out_dir)
    n = 0
    for scen in scenarios:
        base = base_config(scen)
        for name, modify in ABLATIONS:
            d = out_dir / name
            d.mkdir(parents=True, exist_ok=True)
            for seed in SEEDS:
                cfg = copy.deepcopy(base)
                modify(cfg)
                tag = f"{scen}_{SCENARIOS[scen]['gpus']}gpu_s{seed}"
                cfg["output"].update(seed=seed, log_file=f"logs/ablation/{name}/{tag}.log")
                (d / f"{tag}.yaml").write_text(yaml.safe_dump(cfg, sort_keys=False))
                n += 1
    return n


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=str(Path(__file__).resolve().parent.parent / "configs" / "ablation"))
    ap.add_argument("--scenarios", default=",".join(SCENARIOS))
    args = ap.parse_args(argv)
    n = generate(args.out, tuple(args.scenarios.split(",")))
    print(f"wrote {n} configurations ({len(args.scenarios.split(','))} scenario(s) x {len(ABLATIONS)} variants x {len(SEEDS)} seeds)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
