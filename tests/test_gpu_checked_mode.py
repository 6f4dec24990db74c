"""GPU test of checked mode (``RPEG_CHECK_ARGS`` / ``ops.checked.set_enabled``): a whole GRPO step (generation without
graphs, reference pass, policy step) runs with every data-dependent index validated before its launch, and a stray
index is refused BEFORE the kernel that would have followed it is launched."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from rpeg_b200.engine import algorithms as A  # noqa: E402
from rpeg_b200.engine.trainers import GRPOTrainer  # noqa: E402
from rpeg_b200.models.llama import LlamaConfig, LlamaModel  # noqa: E402
from rpeg_b200.ops import checked as C  # noqa: E402
from rpeg_b200.ops import kernels as K  # noqa: E402


@pytest.fixture()
def checked_mode():
    prev = C.set_enabled(True)
    yield
    C.set_enabled(prev)


def test_grpo_step_passes_every_argument_check(cuda_device, checked_mode):
    cfg = LlamaConfig.tiny(n_layers=2)
    tr = GRPOTrainer(cfg, device=cuda_device, samples_per_prompt=4, max_new=24, prompt_len=16, gen_slots=8,
                     kv_budget_bytes=5e8, algo=A.AlgoConfig(kl_coef=0.04, micro_tokens=512, head_chunk=64), seed=3, eos_id=1,
                     use_graphs=False)
    prompts = torch.randint(2, cfg.vocab, (3, 16), dtype=torch.int32)
    rewards = torch.randn(12)
    out = tr.step(prompts, rewards)
    K.check_status()
    assert out["loss"] == out["loss"]


def test_stray_indices_are_refused_before_the_launch(cuda_device, checked_mode):
    cfg = LlamaConfig.tiny(n_layers=1)
    model = LlamaModel(cfg, cuda_device, seed=1)
    table = torch.zeros((cfg.vocab, cfg.d_model), dtype=torch.bfloat16, device=cuda_device)
    ids = torch.tensor([1, cfg.vocab], dtype=torch.int32, device=cuda_device)
    with pytest.raises(C.KernelArgumentError, match=r"rpeg_embed_fwd: ids\[1\]"):
        K.embed_fwd(ids, table)
    x = torch.zeros((4, cfg.d_model), dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(C.KernelArgumentError, match="rpeg_gather_rows"):
        K.gather_rows(x, torch.tensor([0, 4], dtype=torch.int32, device=cuda_device))
    buf = torch.zeros((2, cfg.n_heads * cfg.head_dim), dtype=torch.bfloat16, device=cuda_device)
    pos = torch.tensor([0, model.cos_t.shape[0]], dtype=torch.int32, device=cuda_device)
    with pytest.raises(C.KernelArgumentError, match="rpeg_rope: pos"):
        K.rope_(buf, pos, model.cos_t, model.sin_t, 0, cfg.n_heads, cfg.head_dim)
    torch.cuda.synchronize()
    K.check_status()
    # the same calls with valid indices go through
    K.embed_fwd(torch.tensor([1, cfg.vocab - 1], dtype=torch.int32, device=cuda_device), table)
    K.gather_rows(x, torch.tensor([0, 3], dtype=torch.int32, device=cuda_device))
    torch.cuda.synchronize()


def test_engine_smoke_worker_passes_on_one_gpu(cuda_device, tmp_path, capsys):
    """``runtime.engine_validate``: training step, two-token PPO exercise and checkpoint round trip, as a user runs it."""
    import json

    from rpeg_b200.runtime import engine_validate as ev
    rc = ev.main(["--json", "--ppo-exercise", "--checkpoint-dir", str(tmp_path)])
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rep["schema_version"] == "rpeg.engine_validate.v1"
    assert rc == 0 and rep["ok"], [c for c in rep["checks"] if not c["ok"]]
    assert [c["name"] for c in rep["checks"]] == ["build", "train_step", "ppo_exercise", "checkpoint", "device_status"]


def test_engine_ends_synthetic_rows_at_quantile_lengths(tmp_path, cuda_device):
    """``data.synthetic_response_lengths: quantiles``: every row is ended at the length drawn for it from the
    workload's quantile phases (a natural EOS may still come earlier), so the phases emit rows as the planner assumes."""
    from rpeg_b200.runtime.data import quantile_lengths
    from rpeg_b200.runtime.io import dump_mapping, load_mapping
    from test_gpu_runtime_engine import tiny_job
    run = tiny_job(tmp_path, "grpo", steps=1)
    m = load_mapping(run)
    m.setdefault("data", {}).update(synthetic_response_lengths="quantiles")
    dump_mapping(m, run)
    from rpeg_b200.runtime.compiler import compile_runtime_plan
    from rpeg_b200.runtime.run import execute_compiled
    from rpeg_b200.runtime.trace import read_trace
    compiled = compile_runtime_plan(run)
    res = execute_compiled(compiled, "engine")
    assert res["error"] is None and res["verification"]["ok"], (res["error"], res["verification"]["errors"])
    w = compiled.run_config.workload
    rows = w.batch_size * w.samples_per_prompt
    want = quantile_lengths(rows, w.quantile_tuples(), seed=1)               # data_seed 0, logical step 1
    events = read_trace(tmp_path / "traces/run.jsonl")
    gen = [e for e in events if e["event"] == "finish" and e["node_id"].startswith("g_pi@") and "generated_tokens" in e["counters"]]
    assert len(gen) == 1
    assert 0 < gen[0]["counters"]["generated_tokens"] <= sum(want) < rows * w.generation_length
