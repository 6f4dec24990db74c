"""GPU tests: the runtime graph executed by the engine backend (real kernels) on one GPU, with an
interval checkpoint, a host-side injected failure and a replay of the suffix."""
import json

import pytest
import torch

pytestmark = pytest.mark.gpu

from rpeg_b200.core.types import DeviceSpace  # noqa: E402
from rpeg_b200.runtime import checkpoint as ckpt  # noqa: E402
from rpeg_b200.runtime.compiler import compile_runtime_plan  # noqa: E402
from rpeg_b200.runtime.run import execute_compiled  # noqa: E402
from rpeg_b200.runtime.trace import read_trace  # noqa: E402
from test_runtime_metadata import spread_job  # noqa: E402

TINY = {"layers": 2, "hidden_dim": 256, "ffn_dim": 512, "vocab_size": 512, "head_dim": 128}
WL = {"batch_size": 8, "context_length": 32, "generation_length": 48, "gen_quantiles": [[0.5, 16], [1.0, 48]]}


def tiny_job(tmp_path, algorithm, steps=2, **extra):
    rt = {"default_backend": "engine", "gen_slots": 8, "micro_tokens": 1024}
    rt.update(extra.pop("runtime", {}))
    return spread_job(tmp_path, algorithm, steps=steps, space=DeviceSpace(1, 1, 1), colocate=True, model=TINY, workload=WL,
                      runtime=rt, runtime_hardware={"worker_overhead_bytes": 0}, **extra)


@pytest.mark.parametrize("algorithm", ["grpo", "ppo", "dpo"])
def test_engine_backend_executes_the_graph(tmp_path, cuda_device, algorithm):
    compiled = compile_runtime_plan(tiny_job(tmp_path, algorithm))
    res = execute_compiled(compiled, "engine")
    assert res["error"] is None, res["error"]
    assert res["verification"]["ok"], res["verification"]["errors"]
    events = read_trace(tmp_path / "traces/run.jsonl")
    train = [e for e in events if e["event"] == "finish" and e["node_id"].startswith("t_pi@")]
    assert len(train) == 2 and all(e["counters"]["kernel_launches"] > 0 for e in train)
    assert all(torch.isfinite(torch.tensor(e["counters"]["grad_norm"])) for e in train)
    summary = json.loads((tmp_path / "metrics/summary.json").read_text())
    assert summary["kernel_launches"] > 0 and summary["nonfinite_losses"] == 0
    if algorithm != "dpo":
        assert summary["generation_tokens"] > 0 and summary["generation_emitted_rows"] == 2 * 8 * (2 if algorithm == "grpo" else 1)


def test_engine_checkpoint_replay_restores_weights_and_optimizer(tmp_path, cuda_device):
    run = tiny_job(tmp_path, "grpo", steps=3, checkpoints={"interval_steps": 1},
                   monitoring={"graph_replay_retries": 1, "test_inject_failure_after_checkpoint_step": 2,
                               "test_inject_failure_attempt": 0})
    res = execute_compiled(compile_runtime_plan(run), "engine")
    assert res["error"] is None and res["attempts"] == 2
    rep = res["verification"]
    assert rep["ok"], rep["errors"]
    assert rep["restored_steps"] == [2]
    idx = ckpt.load_index(tmp_path / "checkpoints")
    assert [c["name"] for c in idx["checkpoints"]] == ["step_1", "step_2", "final"]
    for c in idx["checkpoints"]:
        assert ckpt.verify_checkpoint(ckpt.entry_path(tmp_path / "checkpoints", c), c["workers"], hashes=True)["errors"] == []
    w2 = ckpt.load_tensor(tmp_path / "checkpoints/step_2/actor", "weights")
    w3 = ckpt.load_tensor(tmp_path / "checkpoints/final/actor", "weights")
    assert w2.shape == w3.shape and not torch.equal(w2, w3)
    meta = json.loads((tmp_path / "checkpoints/final/actor/meta.json").read_text())
    assert meta["ranks"][0]["extra"] == {"optimizer_step": 3, "version": 3}


def test_engine_runs_update_epochs_over_minibatches(tmp_path, cuda_device):
    """``algorithm.epochs`` x ``algorithm.minibatch_size``: the policy and the critic take one optimizer step per
    minibatch of every epoch (8 rows, minibatches of 4, 2 epochs -> 4 steps per training node)."""
    from rpeg_b200.runtime.io import dump_mapping, load_mapping
    run = tiny_job(tmp_path, "ppo", steps=1)
    m = load_mapping(run)
    m.setdefault("algorithm", {}).update(epochs=2, minibatch_size=4)
    dump_mapping(m, run)
    res = execute_compiled(compile_runtime_plan(run), "engine")
    assert res["error"] is None and res["verification"]["ok"], (res["error"], res["verification"]["errors"])
    events = read_trace(tmp_path / "traces/run.jsonl")
    for prefix in ("t_pi@", "t_V@"):
        fin = [e for e in events if e["event"] == "finish" and e["node_id"].startswith(prefix)]
        assert len(fin) == 1 and fin[0]["counters"]["optimizer_steps"] == 4
