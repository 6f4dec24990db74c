"""Write the planner's scaling-study configurations (PPO, LLaMA-2 shapes) as YAML files.

    python experiments/gen_scaling_configs.py [--out configs/scaling] [--gpus-per-node 8] [--hardware b200|external]

Three studies x four machine sizes x three (generation length, batch) pairs x three staleness variants
= 108 files ``<out>/<study>/<gpus>gpu_t<T>_<variant>.yaml``:
  actor   the actor grows with the machine (7B/13B/34B/70B on 8/16/32/64 GPUs), critic and reward stay 7B
  critic  critic and reward grow, the actor stays 7B
  both    everything grows (16..128 GPUs)
Response lengths follow 50 % by T/4, 85 % by T/2, 100 % by T. ``--hardware b200`` embeds the measured
B200/NVSwitch preset (nodes of 8 GPUs); ``external`` leaves the alpha-beta constants to ``pipeline.py --hw``.
Same experiment matrix as the reference's experiments/gen_scaling_configs.py:23-61, 279-302.
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

import yaml

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

LLAMA2 = {"7b": (32, 4096, 11008), "13b": (40, 5120, 13824), "34b": (48, 8192, 22016), "70b": (80, 8192, 28672)}
LENGTH_BATCH = ((128, 512), (384, 256), (896, 128))
VARIANTS = (("sync", [0], [0]), ("tau1", [1], [0]), ("tau2", [2], [1]))
SEARCH_BUDGET = {8: 55000, 16: 45000, 32: 40000, 64: 30000, 128: 55000}
STUDIES = {
    "actor": ((8, "7b", "7b", "7b"), (16, "13b", "7b", "7b"), (32, "34b", "7b", "7b"), (64, "70b", "7b", "7b")),
    "critic": ((8, "7b", "7b", "7b"), (16, "7b", "13b", "13b"), (32, "7b", "34b", "34b"), (64, "7b", "70b", "70b")),
    "both": ((16, "13b", "13b", "13b"), (32, "13b", "13b", "13b"), (64, "34b", "34b", "13b"), (128, "70b", "70b", "13b")),
}


def model(size: str) -> dict:
    layers, d, f = LLAMA2[size]
    return {"layers": layers, "hidden_dim": d, "ffn_dim": f, "vocab_size": 32000, "head_dim": 128}


def quantiles(T: int) -> list:
    return [[0.5, T // 4], [0.85, T // 2], [1.0, T]]


def hardware_section(gpus: int, gpus_per_node: int, kind: str) -> dict:
    nodes = max(1, gpus // gpus_per_node)
    racks = 2 if nodes >= 16 else 1
    hw = {"racks": racks, "nodes_per_rack": nodes // racks, "gpus_per_node": min(gpus, gpus_per_node)}
    if kind == "b200":
        from rpeg_b200.analytic.hardware import b200_nvswitch
        preset = b200_nvswitch()
        hw.update({k: getattr(preset, k) for k in preset.field_names()})
    return hw


def config(study: str, gpus: int, actor: str, critic: str, reward: str, T: int, B: int, variant: str, tau_a, tau_c,
           gpus_per_node: int, hardware: str) -> dict:
    return {
        "hardware": hardware_section(gpus, gpus_per_node, hardware),
        "models": {"actor": model(actor), "critic": model(critic), "reward": model(reward)},
        "workload": {"batch_size": B, "samples_per_prompt": 1, "context_length": 128, "generation_length": T,
                     "gen_quantiles": quantiles(T)},
        "policy": {"algorithm": "ppo", "allow_ac_share": False},
        "optimizer": {"k_eval": 8, "e_max": SEARCH_BUDGET[gpus], "e_struct": SEARCH_BUDGET[gpus], "k_x": 6, "t_max": 50, "t_init": 0.05,
                      "t_warm": 0.10, "t_min": 0.05, "stag_window": 10, "lambda_ac": 0.0, "score_eps": 1e-4,
                      "staleness_candidates": {"actor": list(tau_a), "critic": list(tau_c)}},
        "output": {"plots": True, "plots_dir": f"figures/runs/scaling/{study}/{gpus}gpu_t{T}_{variant}/",
                   "log_file": f"logs/scaling/{study}/{gpus}gpu_t{T}_{variant}.log"},
    }


def generate(out_dir, gpus_per_node: int = 8, hardware: str = "b200") -> int:
    out_dir = Path(out_dir)
    n = 0
    for study, rows in STUDIES.items():
        (out_dir / study).mkdir(parents=True, exist_ok=True)
        for gpus, actor, critic, reward in rows:
            for T, B in LENGTH_BATCH:
                for variant, tau_a, tau_c in VARIANTS:
                    cfg = config(study, gpus, actor, critic, reward, T, B, variant, tau_a, tau_c, gpus_per_node, hardware)
                    head = f"# scaling study '{study}': {gpus} GPUs, T={T}, B={B}, {variant}; actor {actor}, critic {critic}, reward {reward}\n"
                    (out_dir / study / f"{gpus}gpu_t{T}_{variant}.yaml").write_text(head + yaml.safe_dump(cfg, sort_keys=False))
                    n += 1
    return n


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=str(Path(__file__).resolve().parent.parent / "configs" / "scaling"))
    ap.add_argument("--gpus-per-node", type=int, default=8)
    ap.add_argument("--hardware", default="b200", choices=("b200", "external"))
    args = ap.parse_args(argv)
    print(f"wrote {generate(args.out, args.gpus_per_node, args.hardware)} configurations under {args.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
