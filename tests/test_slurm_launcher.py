"""The Slurm worker-group launcher without Slurm: a stand-in ``srun`` on the test's side starts the step's tasks as local
processes with the environment a real step gives them (``SLURM_PROCID``, ``SLURM_LOCALID``, the node of each task), so the
manifest, the task lookup of ``runtime/pool_entry.py``, idle filler tasks, the stop file and the controller on top of the
launcher are exercised end to end with gloo ranks. Behaviour under test follows RPEG/runtime/launcher.py:212-531 and
RPEG/runtime/semantic_pool_entry.py:47-88."""
import json
import os
import stat
import sys
import textwrap
import time

import pytest

from rpeg_b200.runtime.controller import WorkerGroupController, WorkerGroupSpec
from rpeg_b200.runtime.errors import RuntimeExecutionError
from rpeg_b200.runtime.launcher import RankAssignment, SlurmOptions, SlurmWorkerGroupLauncher, WorkerLaunch

FAKE_SRUN = textwrap.dedent('''\
    #!%(python)s
    # stand-in for srun: starts --ntasks local processes of the command, block distribution over --nodelist
    import os, signal, subprocess, sys, time
    args = sys.argv[1:]
    valued = {"--nodes", "--ntasks", "--ntasks-per-node", "--nodelist", "--distribution", "--export", "--mpi", "--partition",
              "--account", "--time", "--container-image"}
    opts, i = {}, 0
    while i < len(args) and args[i].startswith("--"):
        if args[i] in valued:
            opts[args[i]] = args[i + 1]; i += 2
        else:
            opts[args[i]] = True; i += 1
    cmd, n, per = args[i:], int(opts["--ntasks"]), int(opts["--ntasks-per-node"])
    hosts = opts["--nodelist"].split(",")
    procs = []
    for t in range(n):
        env = dict(os.environ, SLURM_PROCID=str(t), SLURM_LOCALID=str(t %% per), SLURM_NODEID=str(t // per),
                   RPEG_POOL_HOSTNAME=hosts[t // per])
        procs.append(subprocess.Popen(cmd, env=env))
    def forward(sig, frame):
        for p in procs:
            if p.poll() is None:
                p.send_signal(signal.SIGTERM)
    signal.signal(signal.SIGTERM, forward)
    codes = [None] * n
    while any(c is None for c in codes):
        for k, p in enumerate(procs):
            codes[k] = p.poll()
        if any(c not in (None, 0) for c in codes):          # --kill-on-bad-exit
            forward(None, None)
        time.sleep(0.02)
    sys.exit(max(abs(c) for c in codes))
''')


@pytest.fixture
def fake_srun(tmp_path, monkeypatch):
    path = tmp_path / "fake_srun"
    path.write_text(FAKE_SRUN % {"python": sys.executable})
    path.chmod(path.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("SLURM_JOB_ID", "4242")
    return str(path)


def _launch(group, hosts, port, steps=2, log_dir=None, **env):
    assignments, local = [], {}
    for r, h in enumerate(hosts):
        assignments.append(RankAssignment(r, local.get(h, 0), h, None, (group,)))
        local[h] = local.get(h, 0) + 1
    return WorkerLaunch(group, "rpeg_b200.runtime.worker_entry", ("--steps", str(steps), "--backend", "gloo"), assignments,
                        master_port=port, env={k: str(v) for k, v in env.items()}, log_dir=log_dir)


def test_manifest_pads_hosts_with_idle_tasks_and_the_step_is_one_srun(tmp_path):
    opts = SlurmOptions(partition="gpu", account="proj", time_limit="00:30:00", container_image="img.sqsh")
    sl = SlurmWorkerGroupLauncher(tmp_path / "hb", tmp_path / "work", opts)
    gen, train = _launch("gen", ["nodeA", "nodeA"], 29801), _launch("train", ["nodeB.cluster.example"], 29802)
    man = sl.manifest("pool", [gen, train])
    assert man["schema"] == "rpeg.worker_pool.v1" and man["slots_per_host"] == 2
    assert list(man["hosts"]) == ["nodeA", "nodeB"] and [len(v) for v in man["hosts"].values()] == [2, 2]
    idle = [t for t in man["tasks"].values() if t["idle"]]
    assert len(idle) == 1 and idle[0]["hostname"] == "nodeB"
    ranks = {(t["group_id"], t["rank"]): t for t in man["tasks"].values() if not t["idle"]}
    assert set(ranks) == {("gen", 0), ("gen", 1), ("train", 0)}
    assert ranks[("gen", 1)]["env"]["RANK"] == "1" and ranks[("gen", 1)]["env"]["WORLD_SIZE"] == "2"
    assert ranks[("train", 0)]["env"]["MASTER_PORT"] == "29802" and ranks[("train", 0)]["env"]["RPEG_GROUP_ID"] == "train"
    cmd = sl.srun_command(man, tmp_path / "m.json")
    assert cmd[:2] == ["srun", "--overlap"] and cmd[cmd.index("--ntasks") + 1] == "4" and cmd[cmd.index("--ntasks-per-node") + 1] == "2"
    assert cmd[cmd.index("--nodelist") + 1] == "nodeA,nodeB" and cmd[cmd.index("--partition") + 1] == "gpu"
    assert cmd[cmd.index("--account") + 1] == "proj" and cmd[cmd.index("--time") + 1] == "00:30:00"
    assert cmd[cmd.index("--container-image") + 1] == "img.sqsh" and cmd[-4:-2] == ["-m", "rpeg_b200.runtime.pool_entry"]


def test_launcher_refuses_to_run_outside_an_allocation(tmp_path, monkeypatch):
    monkeypatch.delenv("SLURM_JOB_ID", raising=False)
    sl = SlurmWorkerGroupLauncher(tmp_path / "hb", tmp_path / "work")
    with pytest.raises(RuntimeExecutionError, match="inside an existing allocation"):
        sl.launch(_launch("gen", ["nodeA"], 29803))


def test_two_groups_share_one_step_and_the_idle_task_ends_with_the_stop_file(tmp_path, fake_srun):
    sl = SlurmWorkerGroupLauncher(tmp_path / "hb", tmp_path / "work", SlurmOptions(srun=fake_srun))
    logs = str(tmp_path / "logs")
    try:
        sl.launch_pool([_launch("gen", ["nodeA", "nodeA"], 29811, steps=3, log_dir=logs),
                        _launch("train", ["nodeB"], 29812, steps=2, log_dir=logs)], step="pool")
        assert sl.wait_finished("gen", 60.0) == [0, 0] and sl.wait_finished("train", 60.0) == [0]
        step = sl.steps["pool"]
        assert step.poll() is None                                   # the filler task on nodeB keeps the step alive
        assert "sum=" in (tmp_path / "hb" / "gen.rank1.json").read_text()
        sl.stop_step("pool", grace_s=5.0)
        assert step.poll() == 0                                      # ended by the stop file, not by a signal
        assert os.path.exists(os.path.join(logs, "gen.rank0.log"))
    finally:
        sl.stop_all()


def test_a_failing_rank_is_reported_from_its_heartbeat(tmp_path, fake_srun):
    sl = SlurmWorkerGroupLauncher(tmp_path / "hb", tmp_path / "work", SlurmOptions(srun=fake_srun))
    try:
        sl.launch(_launch("gen", ["nodeA", "nodeA"], 29821, RPEG_TEST_FAIL_OPERATION="init", RPEG_TEST_FAIL_RANK=1))
        with pytest.raises(RuntimeExecutionError, match="rank 1 reported an error: RuntimeError: injected failure"):
            sl.wait_ready("gen", 60.0)
        assert "gen" not in sl.step_of                               # a group that failed to come up is torn down
    finally:
        sl.stop_all()


def test_controller_on_the_slurm_launcher_restarts_a_dead_group_as_a_new_step(tmp_path, fake_srun):
    sl = SlurmWorkerGroupLauncher(tmp_path / "hb", tmp_path / "work", SlurmOptions(srun=fake_srun))
    ctl = WorkerGroupController(tmp_path / "hb", restart_retries=1, log_dir=str(tmp_path / "logs"), launcher=sl)
    try:
        ctl.start(WorkerGroupSpec("actor", world=2, table="toy", backend="gloo", master_port=29831, hosts=("nodeA", "nodeA"),
                                  env={"RPEG_TEST_FAIL_OPERATION": "build_model", "RPEG_TEST_FAIL_RANK": "1",
                                       "RPEG_TEST_FAIL_MODE": "exit_after"}))
        ctl.request("actor", "build_model", node_id="build", step=0, payload={"seed": 4, "dim": 8})
        first = sl.steps["actor"]
        deadline = time.monotonic() + 30
        while first.poll() is None and time.monotonic() < deadline:    # rank 1 left: the stand-in ends the step like --kill-on-bad-exit
            time.sleep(0.05)
        assert first.poll() is not None
        got = ctl.request("actor", "checksum", node_id="sum", step=0)   # found dead -> new step -> journal replayed
        assert ctl.restarts == {"actor": 1} and len({r["checksum"] for r in got}) == 1
        assert sl.steps["actor"] is not first
    finally:
        ctl.shutdown()
        sl.stop_all()
