"""Worker groups behind the request tier: requests, restart with journal replay, when a restart is refused.

Everything runs as gloo ranks on the CPU; failures are injected on the host (a rank that leaves between requests or
raises inside one). Behaviour under test follows RPEG/runtime/semantic_controller.py:226-366, 462-538, 594-636.
"""
import time

import pytest

from rpeg_b200.runtime.controller import WorkerGroupController, WorkerGroupSpec, operation_mutates_model
from rpeg_b200.runtime.errors import RuntimeExecutionError

PORT = 29700


def _spec(wid, world, port, **env):
    return WorkerGroupSpec(wid, world=world, table="toy", backend="gloo", master_port=port, env={k: str(v) for k, v in env.items()})


def _wait_gone(ctl, wid, rank, timeout_s=20.0):
    """The injected ``exit_after`` leaves after the reply went out: wait until the process has really ended."""
    alive, deadline = ctl.launcher.alive(wid), time.monotonic() + timeout_s
    while alive(rank) and time.monotonic() < deadline:
        time.sleep(0.02)
    assert not alive(rank)


def _checksum(ctl, wid):
    res = ctl.request(wid, "checksum", node_id="sum", step=0)
    assert len({r["checksum"] for r in res}) == 1           # every rank holds the same model
    return res[0]["checksum"], res[0]["version"]


def test_requests_reach_every_rank_and_journal_keeps_state_ops(tmp_path):
    ctl = WorkerGroupController(tmp_path / "hb", log_dir=str(tmp_path / "logs"))
    try:
        ctl.start(_spec("actor", 2, PORT))
        res = ctl.request("actor", "build_model", node_id="build", step=0, payload={"seed": 3, "dim": 8})
        assert [r["dim"] for r in res] == [8, 8]
        c0, _ = _checksum(ctl, "actor")
        ctl.request("actor", "lm_training_step", node_id="train@1", step=1, payload={"lr": 0.5})
        c1, _ = _checksum(ctl, "actor")
        assert c1 == pytest.approx(c0 - 0.5 * 1.5 * 8)     # mean of the ranks' gradients (1 and 2) times lr, on 8 weights
        assert ctl.journal("actor") == [("build_model", "build")]
        assert not ctl.can_restart("actor")                  # the model was trained and never saved
        with pytest.raises(RuntimeExecutionError, match="unknown operation"):
            ctl.request("actor", "no_such_operation", node_id="x", step=1)
        with pytest.raises(RuntimeExecutionError, match="not been started"):
            ctl.request("actor", "checksum", node_id="x", step=1)   # a failed request aborts the group
    finally:
        ctl.shutdown()


def test_dead_group_is_restarted_and_brought_back_by_replay(tmp_path):
    """Rank 1 leaves right after a weight version was loaded. The next request finds the group dead, starts it again,
    replays ``build_model`` + ``load_weight_version`` and then runs: the state is what it was."""
    path = str(tmp_path / "w1.pt")
    ctl = WorkerGroupController(tmp_path / "hb", restart_retries=1, log_dir=str(tmp_path / "logs"))
    try:
        ctl.start(_spec("actor", 2, PORT + 10, RPEG_TEST_FAIL_OPERATION="load_weight_version", RPEG_TEST_FAIL_RANK=1,
                        RPEG_TEST_FAIL_MODE="exit_after"))
        ctl.request("actor", "build_model", node_id="build", step=0, payload={"seed": 1, "dim": 8})
        ctl.request("actor", "lm_training_step", node_id="train@1", step=1, payload={"lr": 0.25})
        want, _ = _checksum(ctl, "actor")
        ctl.request("actor", "save_weight_version", node_id="save@1", step=1, payload={"path": path, "version": 1})
        assert not ctl.can_restart("actor")                  # saving alone does not make the journal reproduce the model
        ctl.request("actor", "load_weight_version", node_id="load@1", step=1, payload={"path": path})
        assert ctl.can_restart("actor")
        assert ctl.journal("actor") == [("build_model", "build"), ("load_weight_version", "load@1")]
        _wait_gone(ctl, "actor", 1)
        got, version = _checksum(ctl, "actor")              # rank 1 is gone by now: restart + replay happen in here
        assert ctl.restarts == {"actor": 1}
        assert (got, version) == (pytest.approx(want), 1)
        ctl.request("actor", "lm_training_step", node_id="train@2", step=2, payload={"lr": 0.25})
        assert _checksum(ctl, "actor")[0] == pytest.approx(want - 0.25 * 1.5 * 8)
    finally:
        ctl.shutdown()


def test_restart_is_refused_after_an_unsaved_training_step(tmp_path):
    ctl = WorkerGroupController(tmp_path / "hb", restart_retries=2, log_dir=str(tmp_path / "logs"))
    try:
        ctl.start(_spec("actor", 2, PORT + 20, RPEG_TEST_FAIL_OPERATION="lm_training_step", RPEG_TEST_FAIL_RANK=0,
                        RPEG_TEST_FAIL_MODE="exit_after"))
        ctl.request("actor", "build_model", node_id="build", step=0, payload={"seed": 1})
        ctl.request("actor", "lm_training_step", node_id="train@1", step=1)
        _wait_gone(ctl, "actor", 0)
        with pytest.raises(RuntimeExecutionError, match="not restarted because its model was changed") as err:
            ctl.request("actor", "checksum", node_id="sum", step=1)
        assert "rank 0" in str(err.value) and "heartbeats=" in str(err.value)
        assert ctl.restarts == {}
    finally:
        ctl.shutdown()


def test_restart_budget_and_failure_inside_a_request(tmp_path):
    """A rank raising INSIDE a request fails that request and aborts the group (no silent retry of a request whose
    effects are unknown); with ``restart_retries=0`` a dead group is never started again."""
    ctl = WorkerGroupController(tmp_path / "hb", restart_retries=0, log_dir=str(tmp_path / "logs"))
    try:
        ctl.start(_spec("critic", 2, PORT + 30, RPEG_TEST_FAIL_OPERATION="checksum", RPEG_TEST_FAIL_RANK=1, RPEG_TEST_FAIL_MODE="raise"))
        ctl.request("critic", "build_model", node_id="build", step=0)
        with pytest.raises(RuntimeExecutionError, match="injected failure in checksum.*worker group aborted"):
            ctl.request("critic", "checksum", node_id="sum", step=0)
        ctl.start(_spec("critic2", 1, PORT + 40, RPEG_TEST_FAIL_OPERATION="build_model", RPEG_TEST_FAIL_MODE="exit_after"))
        ctl.request("critic2", "build_model", node_id="build", step=0)
        _wait_gone(ctl, "critic2", 0)
        with pytest.raises(RuntimeExecutionError, match="restarts are exhausted"):
            ctl.request("critic2", "checksum", node_id="sum", step=0)
    finally:
        ctl.shutdown()


def test_paired_requests_check_both_groups_first_and_abort_both_on_failure(tmp_path):
    path = str(tmp_path / "v.pt")
    ctl = WorkerGroupController(tmp_path / "hb", restart_retries=1, log_dir=str(tmp_path / "logs"))
    try:
        ctl.start(_spec("train", 1, PORT + 50))
        ctl.start(_spec("gen", 1, PORT + 60, RPEG_TEST_FAIL_OPERATION="build_model", RPEG_TEST_FAIL_MODE="exit_after"))
        ctl.request_many([("train", "build_model", "b", 0, {"seed": 5}, 30.0), ("gen", "build_model", "b", 0, {"seed": 6}, 30.0)])
        ctl.request("train", "save_weight_version", node_id="save", step=0, payload={"path": path, "version": 7})
        _wait_gone(ctl, "gen", 0)
        # "gen" died after building: the paired call restarts it (replaying its build) before sending either half
        out = ctl.request_many([("train", "checksum", "s", 0, {}, 30.0), ("gen", "load_weight_version", "l", 0, {"path": path}, 30.0)])
        assert ctl.restarts == {"gen": 1} and out["gen"][0]["version"] == 7
        assert _checksum(ctl, "gen")[0] == pytest.approx(out["train"][0]["checksum"])
        with pytest.raises(RuntimeExecutionError, match="all participants aborted"):
            ctl.request_many([("train", "checksum", "s", 1, {}, 30.0), ("gen", "no_such_operation", "x", 1, {}, 30.0)])
        for wid in ("train", "gen"):
            with pytest.raises(RuntimeExecutionError, match="not been started"):
                ctl.request(wid, "checksum", node_id="s", step=1)
    finally:
        ctl.shutdown()


def test_a_group_whose_controller_is_gone_shuts_itself_down(tmp_path):
    ctl = WorkerGroupController(tmp_path / "hb", log_dir=str(tmp_path / "logs"))
    try:
        ctl.start(_spec("actor", 2, PORT + 70))
        ctl.request("actor", "build_model", node_id="build", step=0)
        ctl._groups["actor"].client.close()                       # the controller's side of the connection disappears
        beats = ctl.launcher.control.wait_for_state("actor", 2, ("finished",), 30.0)
        assert [b.state for b in beats] == ["finished", "finished"]
        assert ctl.launcher.wait_finished("actor", 10.0) == [0, 0]
    finally:
        ctl.launcher.stop_all()


def test_which_operations_count_as_mutating():
    assert operation_mutates_model("lm_training_step") and operation_mutates_model("policy_train_step")
    assert not operation_mutates_model("checksum") and not operation_mutates_model("generate")
