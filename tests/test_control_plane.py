"""CPU tests of the control plane: heartbeats, the local launcher and failure detection with gloo
ranks. Every failure is made on the host (a rank that raises, never becomes ready or exits)."""
import os
import threading
import time

import pytest

from rpeg_b200.runtime.control import ControlPlane, Heartbeat, HeartbeatStore
from rpeg_b200.runtime.errors import RuntimeExecutionError
from rpeg_b200.runtime.launcher import (LocalWorkerGroupLauncher, WorkerLaunch, rank_environment, single_node_assignments,
                                        torchrun_command)

_PORT = [29600 + (os.getpid() % 200)]


def launch(tmp_path, world=2, steps=3, env=None, **kw):
    _PORT[0] += 1
    l = LocalWorkerGroupLauncher(tmp_path / "hb")
    wl = WorkerLaunch("grp", "rpeg_b200.runtime.worker_entry", ["--steps", str(steps), *kw.pop("args", [])],
                      single_node_assignments(world, ("actor",), cuda=False), master_port=_PORT[0], env=env or {},
                      log_dir=str(tmp_path / "logs"))
    l.launch(wl)
    return l


def test_heartbeat_store_and_wait(tmp_path):
    store = HeartbeatStore(tmp_path)
    cp = ControlPlane(store, poll_s=0.005)
    assert store.read("w", 0) is None
    a = store.write("w", 0, "starting")
    b = store.write("w", 0, "ready", step=1)
    assert (a.sequence, b.sequence) == (1, 2) and store.read("w", 0).state == "ready"
    with pytest.raises(ValueError):
        Heartbeat("w", 0, "bogus")
    with pytest.raises(RuntimeExecutionError, match="timed out"):
        cp.wait_for_state("w", 2, ("ready",), timeout_s=0.05)
    threading.Timer(0.05, lambda: store.write("w", 1, "ready")).start()
    assert [h.state for h in cp.wait_for_state("w", 2, ("ready",), timeout_s=2.0)] == ["ready", "ready"]
    store.write("w", 1, "error", message="boom")
    with pytest.raises(RuntimeExecutionError, match="boom"):
        cp.wait_for_state("w", 2, ("finished",), timeout_s=1.0)
    with pytest.raises(RuntimeExecutionError, match="boom"):
        cp.assert_healthy("w", 2)


def test_rank_environment_and_torchrun_line(tmp_path):
    wl = WorkerLaunch("g", "m", (), single_node_assignments(4, ("actor", "critic")), master_port=1234)
    env = rank_environment(wl, wl.assignments[2], str(tmp_path))
    assert (env["MASTER_ADDR"], env["MASTER_PORT"], env["WORLD_SIZE"], env["RANK"], env["LOCAL_RANK"]) == ("127.0.0.1", "1234", "4", "2", "2")
    assert '"worker_ids": ["actor", "critic"]' in env["RPEG_RANK_ASSIGNMENTS_JSON"]
    cmd = torchrun_command("rpeg_b200.runtime.run", ["--config", "run.yaml"], 8)
    assert "--nproc-per-node=8" in cmd and cmd[cmd.index("--master-addr") + 1] == "127.0.0.1"


def test_gloo_ranks_run_to_completion(tmp_path):
    l = launch(tmp_path, world=2, steps=3)
    try:
        l.wait_ready("grp", timeout_s=60)
        assert l.wait_finished("grp", timeout_s=60) == [0, 0]
        assert [l.store.read("grp", r).state for r in range(2)] == ["finished", "finished"]
    finally:
        l.stop_all()


@pytest.mark.parametrize("op,match", [("init", "injected failure during initialisation"), ("step", "injected failure before step 2"),
                                      ("exit", "exit codes")])
def test_rank_failure_is_detected_and_the_group_is_aborted(tmp_path, op, match):
    env = {"RPEG_TEST_FAIL_OPERATION": op, "RPEG_TEST_FAIL_RANK": "1", "RPEG_TEST_FAIL_STEP": "2"}
    l = launch(tmp_path, world=2, steps=50, env=env, args=["--step-sleep", "0.05", "--collective-timeout", "5"])
    try:
        with pytest.raises(RuntimeExecutionError, match=match):
            l.wait_ready("grp", timeout_s=60)
            l.wait_finished("grp", timeout_s=60)
        assert "grp" not in l.procs                      # torn down as a whole
    finally:
        l.stop_all()
    hb0 = HeartbeatStore(tmp_path / "hb").read("grp", 0)
    # rank 0 may have been torn down before it wrote its first heartbeat; if it wrote one, it never reached "finished"
    assert hb0 is None or hb0.state in ("starting", "ready", "running", "stopped", "error")


def test_rank_that_never_becomes_ready_times_out(tmp_path):
    l = launch(tmp_path, world=2, steps=2, env={"RPEG_TEST_FAIL_OPERATION": "never_ready", "RPEG_TEST_FAIL_RANK": "0"},
               args=["--collective-timeout", "3"])
    t0 = time.monotonic()
    try:
        with pytest.raises(RuntimeExecutionError, match="timed out|reported an error"):
            l.wait_ready("grp", timeout_s=4.0)
        assert time.monotonic() - t0 < 30 and "grp" not in l.procs
    finally:
        l.stop_all()
