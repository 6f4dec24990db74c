"""Reference arm of ``bench.py``: runs the reference framework's own code, from the copy under
``baseline/_ref`` (``baseline/install_ref.py``), through its own command lines, in subprocesses.

Two entry points:

``planner_arm``   the reference's ``pipeline.py --config <yaml>`` (analytical plan search on CPU); reports the
                  search wall time it prints and the throughput of its optimized plan.
``torch_arm``     the reference's tensor path on one GPU: ``python -m runtime.job_plan`` on a job file that names
                  a Hugging Face Llama directory, then ``python -m runtime.run`` with
                  ``runtime.default_backend: torch_grpo`` (``TorchPPOGraphHandler``, Hugging Face
                  ``AutoModelForCausalLM`` + ``generate`` + ``torch.optim.AdamW``); per-step times come from the
                  trace the run writes. The model directory holds random-init weights of the benchmark's
                  architecture, a word-level tokenizer over the same vocabulary and prompts of the benchmark's
                  length, all written here because there is no network.

Nothing of this framework's engine, kernels or models is imported on these paths. Whatever the reference raises
is passed on verbatim in the ``unavailable`` line.
"""
from __future__ import annotations

import json
import os
import re
import subprocess
import sys
import time
from pathlib import Path
from typing import Dict, Optional

HERE = Path(__file__).resolve().parent
REF = HERE / "_ref"


class ReferenceUnavailable(RuntimeError):
    pass


def _env() -> Dict[str, str]:
    sys.path.insert(0, str(HERE))
    try:
        from install_ref import env_for_reference
    finally:
        sys.path.pop(0)
    return env_for_reference()


def ensure_installed() -> None:
    if (REF / ".installed").exists():
        return
    sys.path.insert(0, str(HERE))
    try:
        from install_ref import install
        install(Path("/root/reference"))
    except Exception as exc:  # noqa: BLE001
        raise ReferenceUnavailable(f"no reference copy under baseline/_ref and none could be made: {type(exc).__name__}: {exc}")
    finally:
        sys.path.pop(0)


def _tail(text: str, n: int = 6) -> str:
    lines = [ln.strip() for ln in text.strip().splitlines() if ln.strip()]
    return " | ".join(lines[-n:])[-900:]


# ------------------------------------------------------------------------------------------ planner
def planner_arm(config_yaml: Path, timeout_s: float = 900.0) -> Dict[str, float]:
    """Reference plan search on ``config_yaml``. Returns the numbers of its result table."""
    ensure_installed()
    t0 = time.perf_counter()
    res = subprocess.run([sys.executable, str(REF / "pipeline.py"), "--config", str(config_yaml)], cwd=str(REF), env=_env(),
                         capture_output=True, text=True, timeout=timeout_s)
    wall = time.perf_counter() - t0
    if res.returncode != 0:
        raise ReferenceUnavailable(f"reference pipeline.py exited {res.returncode}: {_tail(res.stderr or res.stdout)}")
    out = res.stdout
    m_thr = re.search(r"Throughput \(tokens/s\)\s+(\S+)\s+(\S+)\s+(\S+)", out)
    m_mk = re.search(r"Makespan \(s\)\s+(\S+)\s+(\S+)\s+(\S+)", out)
    m_wall = re.search(r"wall time\s+([0-9.]+)s", out)
    if not (m_thr and m_mk):
        raise ReferenceUnavailable(f"reference pipeline.py printed no result table: {_tail(out)}")
    return {"greedy_tokens_per_s": float(m_thr.group(1)), "heuristic_tokens_per_s": float(m_thr.group(2)),
            "optimized_tokens_per_s": float(m_thr.group(3)), "optimized_makespan_s": float(m_mk.group(3)),
            "search_wall_s": float(m_wall.group(1)) if m_wall else wall, "process_wall_s": wall}


# ------------------------------------------------------------------------------------------ tensor path
def write_assets(root: Path, *, layers: int, hidden: int, ffn: int, heads: int, kv_heads: int, vocab: int, max_pos: int,
                 n_prompts: int, prompt_len: int, seed: int = 42) -> Path:
    """A Hugging Face Llama directory (config, random-init bf16 safetensors, word-level tokenizer) and a prompt file."""
    import torch
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import LlamaConfig, LlamaForCausalLM, PreTrainedTokenizerFast

    model_dir = root / "model"
    model_dir.mkdir(parents=True, exist_ok=True)
    words = ["<pad>", "<s>", "</s>"] + [f"w{i}" for i in range(3, vocab)]
    tok = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<pad>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<s>", eos_token="</s>", pad_token="<pad>", unk_token="<pad>")
    fast.save_pretrained(model_dir)
    cfg = LlamaConfig(vocab_size=vocab, hidden_size=hidden, intermediate_size=ffn, num_hidden_layers=layers,
                      num_attention_heads=heads, num_key_value_heads=kv_heads, max_position_embeddings=max_pos,
                      rms_norm_eps=1e-5, tie_word_embeddings=False, bos_token_id=1, eos_token_id=2, pad_token_id=0,
                      torch_dtype="bfloat16")
    torch.manual_seed(seed)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    with torch.device(dev):
        model = LlamaForCausalLM(cfg).to(torch.bfloat16)
    model.save_pretrained(model_dir, safe_serialization=True)
    del model
    if dev == "cuda":
        torch.cuda.empty_cache()
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(3, vocab, (n_prompts, prompt_len), generator=g)
    with (root / "prompts.jsonl").open("w") as f:
        for row in ids.tolist():
            f.write(json.dumps({"prompt": " ".join(f"w{t}" for t in row)}) + "\n")
    return model_dir


def torch_arm(*, algo: str, model: Dict[str, int], prompts: int, samples_per_prompt: int, prompt_len: int, max_new: int,
              quantiles, steps: int, warmup: int, workdir: Path, hw_memory_bytes: float = 1.9e11,
              timeout_s: float = 3000.0) -> Dict[str, float]:
    """Run ``warmup + steps`` iterations of the reference's single-device torch backend; time the last ``steps``."""
    import yaml

    ensure_installed()
    if algo != "grpo":
        raise ReferenceUnavailable(f"the reference arm drives the GRPO torch backend; '{algo}' is not wired")
    workdir.mkdir(parents=True, exist_ok=True)
    total = warmup + steps
    deadline = time.perf_counter() + timeout_s          # writing the model directory counts
    model_dir = write_assets(workdir, n_prompts=prompts * total, prompt_len=prompt_len, max_pos=prompt_len + max_new + 8, **model)
    job = {
        "run_id": "ref-grpo",
        "policy": {"algorithm": "grpo", "tau": {"actor": 0}},
        "hardware": {"racks": 1, "nodes_per_rack": 1, "gpus_per_node": 1, "flops_per_gpu": 1.35e15, "memory_per_gpu": hw_memory_bytes,
                     "memory_bandwidth": 6.5e12},
        "device_space": {"racks": 1, "nodes_per_rack": 1, "gpus_per_node": 1},
        "models": {"actor": {"source": "local", "checkpoint_path": str(model_dir), "dtype": "bf16"},
                   "reference": {"source": "actor"}, "reward": {"source": "actor"}},
        "workload": {"batch_size": prompts, "samples_per_prompt": samples_per_prompt, "context_length": prompt_len,
                     "generation_length": max_new, "gen_quantiles": [list(q) for q in quantiles] if quantiles else None},
        "algorithm": {"do_sample": True, "temperature": 1.0, "top_p": 1.0, "top_k": 0, "seed": 42, "kl_coef": 0.04},
        "training": {"max_steps": total},
        "optimizer": {"k_eval": 1, "staleness_candidates": {"actor": [0]}},
        "optimizer_runtime": {"distributed_optimizer": "none"},
        "runtime": {"default_backend": "torch_grpo"},
        "data": {"train_prompts": str(workdir / "prompts.jsonl")},
        "checkpoints": {"save_final": False, "interval_steps": 10 ** 9},
    }
    (workdir / "job.yaml").write_text(yaml.safe_dump(job, sort_keys=False))
    env = _env()
    out_dir = workdir / "job"

    def left() -> float:
        return max(5.0, deadline - time.perf_counter())

    try:
        res = subprocess.run([sys.executable, "-m", "runtime.job_plan", "--config", str(workdir / "job.yaml"), "--out-dir", str(out_dir)],
                             cwd=str(REF), env=env, capture_output=True, text=True, timeout=left())
    except subprocess.TimeoutExpired as exc:
        raise ReferenceUnavailable(f"reference runtime.job_plan did not finish within {timeout_s:.0f} s") from exc
    if res.returncode != 0 or not (out_dir / "run.yaml").exists():
        raise ReferenceUnavailable(f"reference runtime.job_plan exited {res.returncode}: {_tail(res.stderr or res.stdout)}")
    t0 = time.perf_counter()
    try:
        res = subprocess.run([sys.executable, "-m", "runtime.run", "--config", str(out_dir / "run.yaml")], cwd=str(REF), env=env,
                             capture_output=True, text=True, timeout=left())
    except subprocess.TimeoutExpired as exc:
        raise ReferenceUnavailable(f"reference runtime.run (torch_grpo backend, 1 GPU) did not finish {total} step(s) of this configuration "
                                   f"within the {timeout_s:.0f} s given to the reference arm") from exc
    wall = time.perf_counter() - t0
    if res.returncode != 0:
        raise ReferenceUnavailable(f"reference runtime.run (torch_grpo backend, 1 GPU) exited {res.returncode}: {_tail(res.stderr or res.stdout)}")
    run_cfg = yaml.safe_load((out_dir / "run.yaml").read_text())
    return _step_times(Path(run_cfg["runtime"]["trace_path"]), total, warmup, wall, prompts * samples_per_prompt)


def _step_times(trace_path: Path, total: int, warmup: int, wall: float, samples_per_step: int) -> Dict[str, float]:
    """Per-step wall time from the reference's own trace: first node start to last node finish of a logical step."""
    spans: Dict[int, list] = {}
    gen_tokens = 0
    for line in trace_path.read_text().splitlines():
        if not line.strip():
            continue
        ev = json.loads(line)
        step = ev.get("logical_step", ev.get("step"))
        t = ev.get("time", ev.get("timestamp", ev.get("ts")))
        if step is None or t is None:
            continue
        span = spans.setdefault(int(step), [float(t), float(t)])
        span[0], span[1] = min(span[0], float(t)), max(span[1], float(t))
        counters = ev.get("counters") or {}
        if int(step) > warmup and "generated_tokens" in counters:
            gen_tokens += int(counters["generated_tokens"])
    timed = [s for s in sorted(spans) if s > warmup]
    if not timed:
        secs = wall * (total - warmup) / max(total, 1)
        n = total - warmup
    else:
        secs = spans[timed[-1]][1] - spans[timed[0]][0]
        n = len(timed)
    return {"seconds": secs, "steps": n, "samples_per_s": samples_per_step * n / secs, "gen_tokens_per_s": gen_tokens / secs if gen_tokens else None,
            "process_wall_s": wall}
