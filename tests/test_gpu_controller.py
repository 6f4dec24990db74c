"""The request tier with the engine table on a GPU: a worker group that holds ``LlamaModel`` + ``AdamW`` is trained,
its weights published and loaded, the process ends between requests (on the host, nothing in flight) and the
controller brings a new one back to the same weights by replaying the journal."""
import dataclasses
import time

import pytest
import torch

from rpeg_b200.runtime.controller import WorkerGroupController, WorkerGroupSpec

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")
def test_engine_group_restart_replays_build_and_weight_version(tmp_path):
    from rpeg_b200.models.llama import LlamaConfig
    cfg = dataclasses.asdict(LlamaConfig.tiny())
    path = str(tmp_path / "actor_v1.pt")
    ctl = WorkerGroupController(tmp_path / "hb", restart_retries=1, log_dir=str(tmp_path / "logs"), ready_timeout_s=300.0)
    try:
        ctl.start(WorkerGroupSpec("actor", world=1, table="engine", backend="nccl", master_port=29790, cuda=True,
                                  env={"RPEG_TEST_FAIL_OPERATION": "load_weight_version", "RPEG_TEST_FAIL_MODE": "exit_after"}))
        ctl.request("actor", "build_model", node_id="build", step=0, payload={"config": cfg, "seed": 2, "lr": 1e-3}, timeout_s=300.0)
        c0 = ctl.request("actor", "checksum", node_id="sum", step=0)[0]["checksum"]
        out = ctl.request("actor", "lm_training_step", node_id="train@1", step=1, payload={"seed": 1, "batch": 4}, timeout_s=300.0)[0]
        assert out["loss"] == out["loss"] and out["grad_norm"] > 0
        c1 = ctl.request("actor", "checksum", node_id="sum", step=1)[0]["checksum"]
        assert c1 != c0
        ctl.request("actor", "save_weight_version", node_id="save@1", step=1, payload={"path": path, "version": 1})
        ctl.request("actor", "load_weight_version", node_id="load@1", step=1, payload={"path": path})
        alive, deadline = ctl.launcher.alive("actor"), time.monotonic() + 30
        while alive(0) and time.monotonic() < deadline:
            time.sleep(0.05)
        got = ctl.request("actor", "checksum", node_id="sum", step=1, timeout_s=300.0)[0]
        assert ctl.restarts == {"actor": 1}
        assert got["version"] == 1 and got["checksum"] == pytest.approx(c1, rel=1e-6)
    finally:
        ctl.shutdown()
