"""GPU tests of tensor-parallel decoding (``models/tp_decode.py``, ``csrc/tp_decode.cu``): the self test of
``parallel/tp_decode_selftest.py`` on one rank (the same kernels with a world of one) and, where the box has them, on
two ranks with plain peer access and with the NVLS multicast mapping, plus the tiny benchmark with tensor-parallel
generation."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

from test_gpu_multi import ROOT, _last_json, _torchrun  # noqa: E402


def test_tp_decode_selftest_one_rank():
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, "-m", "rpeg_b200.parallel.tp_decode_selftest"], cwd=ROOT, env=env, capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    rep = _last_json(r.stdout)
    assert rep["ok"] and rep["world"] == 1 and rep["decode_step_max_rel_err"] < 4e-2, rep


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("comm", ["peer", "auto"])
def test_tp_decode_selftest_two_ranks(comm):
    r = _torchrun(2, 29571 if comm == "peer" else 29572, "-m", "rpeg_b200.parallel.tp_decode_selftest", "--comm", comm)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    rep = _last_json(r.stdout)
    assert rep["ok"] and rep["world"] == 2 and rep["gen_identical_on_ranks"], rep


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_bench_tiny_two_ranks_tensor_parallel_generation():
    r = _torchrun(2, 29573, "bench.py", "--config", "grpo_tiny", "--gpus", "2", "--steps", "2", "--warmup", "3", "--gen-parallel", "tp")
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = _last_json(r.stdout)
    assert line["n_gpus"] == 2 and line["value"] > 0 and "tp2" in line["config"]["parallelism"] and line["reshard_us"] > 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_bench_falls_back_to_data_parallel_generation_when_the_start_up_check_fails(monkeypatch):
    """``--gen-parallel auto`` checks the tensor-parallel decode step against the whole model before the run; a failed
    check (forced here on the host, nothing faults) must leave a working data-parallel benchmark, not a failed job."""
    monkeypatch.setenv("RPEG_BENCH_FORCE_TP_FALLBACK", "1")
    r = _torchrun(2, 29574, "bench.py", "--config", "grpo_tiny", "--gpus", "2", "--steps", "2", "--warmup", "3")
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = _last_json(r.stdout)
    assert line["n_gpus"] == 2 and line["value"] > 0 and line["config"]["parallelism"] == "dp2", line["config"]
    assert "generating data parallel" in r.stderr


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs four GPUs")
def test_bench_tiny_four_ranks_generation_in_two_tensor_parallel_groups():
    """Generation layout (2, 1, 2): two groups of two ranks, each group decodes the rows of its own prompts."""
    r = _torchrun(4, 29575, "bench.py", "--config", "grpo_tiny", "--gpus", "4", "--steps", "2", "--warmup", "3", "--gen-tp-size", "2")
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = _last_json(r.stdout)
    assert line["n_gpus"] == 4 and line["value"] > 0 and "dp2 x tp2" in line["config"]["parallelism"], line["config"]
    assert line["last_step"]["grad_norm"] > 0 and line["last_step"]["samples"] > 0
