"""Predicted time of one benchmark iteration from the analytical cost model.

``predict_step_seconds(spec, n_gpus, parallelism=...)`` builds the workload of a ``bench.py`` configuration
(prompts, samples per prompt, prompt and generation lengths, length quantiles, model shape), the plan the benchmark
executes on ``n_gpus`` GPUs of one node (every vertex data parallel; the generation vertex tensor parallel when the
benchmark generates that way) and the hardware constants measured on this pool (``configs/hw_b200_measured.yaml``
over the ``b200_nvswitch`` preset), then runs the compiler's own pipeline: unroll, lower, cost model, list scheduler.
The makespan of one iteration is the prediction that the benchmark sets against its measured step
(``cost_model_err``). Reference for the pipeline: pipeline.py:1247-1765 (evaluate a plan), RPEG/model/cost.py:34-130.
"""
from __future__ import annotations

from pathlib import Path
from typing import Any, Dict, Optional

_ROOT = Path(__file__).resolve().parent.parent.parent
_SHAPES = {
    "llama7b": {"layers": 32, "hidden_dim": 4096, "ffn_dim": 11008, "vocab_size": 32000, "head_dim": 128},
    "llama13b": {"layers": 40, "hidden_dim": 5120, "ffn_dim": 13824, "vocab_size": 32000, "head_dim": 128},
    "tiny": {"layers": 2, "hidden_dim": 256, "ffn_dim": 512, "vocab_size": 512, "head_dim": 128},
}


def bench_job_mapping(spec: Dict[str, Any], n_gpus: int, *, gen_slots: int = 256, kv_budget_bytes: float = 56e9,
                      micro_tokens: int = 16384, hw_file: Optional[str] = None, recompute_fraction: float = 1.0) -> Dict[str, Any]:
    """The benchmark configuration as a planner job mapping (the keys of ``runtime.job_plan`` job files)."""
    algo = {"grpo_async": "grpo"}.get(spec["algo"], spec["algo"])
    hw_path = Path(hw_file) if hw_file else _ROOT / "configs" / "hw_b200_measured.yaml"
    hardware: Dict[str, Any] = {"preset": "b200_nvswitch", "memory_per_gpu": 192e9, "expected_lengths": 1.0}
    if hw_path.exists():
        hardware["file"] = str(hw_path)
    if int(spec.get("k", 1)) > 1:
        hardware["gen_shared_prompt_cost"] = 0.51        # K samples alias their prompt's KV pages (L2 hits)
    models: Dict[str, Any] = {"actor": dict(_SHAPES[spec["model"]]), "reference": {"source": "actor"}}
    if algo == "ppo":
        models["critic"] = {"source": "actor"}
        models["reward"] = dict(_SHAPES["llama7b" if spec["model"] == "llama13b" else spec["model"]])
    workload: Dict[str, Any] = {"batch_size": int(spec["prompts"]), "samples_per_prompt": int(spec["k"]),
                                "context_length": int(spec["prompt_len"]), "generation_length": int(spec["max_new"])}
    if spec.get("quantiles"):
        workload["gen_quantiles"] = [list(q) for q in spec["quantiles"]]
    return {"run_id": "bench-prediction", "policy": {"algorithm": algo}, "hardware": hardware,
            "device_space": {"racks": 1, "nodes_per_rack": 1, "gpus_per_node": int(n_gpus)}, "models": models, "workload": workload,
            "optimizer": {"k_eval": 1}, "optimizer_runtime": {"distributed_optimizer": "zero1", "activation_checkpointing": float(recompute_fraction)},
            "runtime_hardware": {"worker_overhead_bytes": 2 ** 30, "memory_reserve_fraction": 0.02,
                                 "kv_cache_budget_bytes": float(kv_budget_bytes), "activation_token_cap": int(micro_tokens)},
            "runtime": {"default_backend": "engine", "gen_slots": int(gen_slots), "micro_tokens": int(micro_tokens)}}


def predict_step_seconds(spec: Dict[str, Any], n_gpus: int, *, parallelism: str = "", hw_file: Optional[str] = None,
                         gen_slots: int = 256, recompute_fraction: float = 1.0) -> Dict[str, Any]:
    """``recompute_fraction``: share of the layers whose forward pass runs again in the backward pass (1 = all)."""
    from ..core.types import Allocation, Role
    from ..ir.plan import ExecutionPlan
    from ..ir.templates import build_rpeg
    from ..passes.lower import ExecNodeType
    from ..runtime import job_plan as J
    from ..search.evaluate import Configuration

    cfg = bench_job_mapping(spec, n_gpus, gen_slots=gen_slots, hw_file=hw_file, recompute_fraction=recompute_fraction)
    base = _ROOT / "configs"
    space, hw, suite = J.job_device_space(cfg), J.job_hardware(cfg, base), J.job_suite(cfg)
    workload, policy = J.job_workload(cfg, base), J.job_memory_policy(cfg)
    rpeg = build_rpeg(cfg["policy"]["algorithm"], suite, workload)
    g = space.num_devices()
    import re
    m_tp = re.search(r"generation (?:dp(\d+) x )?tp(\d+)", parallelism)
    gen_tp = m_tp is not None
    gen_pi = (int(m_tp.group(1) or 1), 1, int(m_tp.group(2))) if gen_tp else None
    full = Allocation((0, 0, 0), (space.R, space.N, space.G))
    plan = ExecutionPlan()
    for v in rpeg.vertices:
        plan.sigma[v.id], plan.mb[v.id] = full, 1
        plan.pi[v.id] = gen_pi if (gen_tp and v.kind.role is Role.GENERATION) else (g, 1, 1)
    trace, lowered = J.predicted_schedule(Configuration(rpeg, plan, space), suite, workload, hw, 1, policy)
    phases: Dict[str, float] = {}
    for n in lowered.nodes:
        key = n.role.value if n.kind is ExecNodeType.OP else n.kind.value
        phases[key] = phases.get(key, 0.0) + float(trace.finish[n] - trace.start[n])
    return {"step_s": float(trace.makespan()), "phases_s": {k: round(v, 4) for k, v in phases.items()},
            "hardware": "b200_nvswitch preset + configs/hw_b200_measured.yaml", "plan": {v: list(p) for v, p in plan.pi.items()}}
