"""Pipeline-parallel host logic: the 1F1B order, its activation bound, and the per-stage parameter tables."""
import pytest

from rpeg_b200.models.llama import LlamaConfig, ParamLayout, stage_layers
from rpeg_b200.parallel.pp import one_f_one_b, peak_live_microbatches
from rpeg_b200.parallel.reshard import stage_of


@pytest.mark.parametrize("p,m", [(1, 3), (2, 4), (4, 8), (4, 2), (8, 8), (3, 1)])
def test_one_f_one_b_is_a_valid_schedule(p, m):
    orders = [one_f_one_b(s, p, m) for s in range(p)]
    for s, order in enumerate(orders):
        assert sorted(i for k, i in order if k == "F") == list(range(m))
        assert sorted(i for k, i in order if k == "B") == list(range(m))
        seen_f = set()
        for k, i in order:
            if k == "F":
                seen_f.add(i)
            else:
                assert i in seen_f                       # backward only after its own forward
        assert peak_live_microbatches(s, p, m) == min(p - s, m)
    # Simulate: an operation may run once its input exists (forward from the stage before, backward from the
    # stage after). Every stage executes its list in order; the whole thing must finish (no circular wait).
    pos = [0] * p
    done = set()
    progressed = True
    while progressed:
        progressed = False
        for s in range(p):
            if pos[s] == len(orders[s]):
                continue
            k, i = orders[s][pos[s]]
            ready = (k == "F" and (s == 0 or ("F", s - 1, i) in done)) or (k == "B" and (s == p - 1 or ("B", s + 1, i) in done))
            if ready:
                done.add((k, s, i))
                pos[s] += 1
                progressed = True
    assert all(pos[s] == len(orders[s]) for s in range(p))


def test_stage_layers_cover_all_layers_and_match_reshard_rule():
    cfg = LlamaConfig.tiny(n_layers=7)
    for pp in (1, 2, 3, 7):
        covered = []
        for s in range(pp):
            lo, hi = stage_layers(cfg.n_layers, (s, pp))
            covered += list(range(lo, hi))
            for l in range(lo, hi):
                assert stage_of(cfg, f"l{l}.wqkv", pp) == s
        assert covered == list(range(cfg.n_layers))
    with pytest.raises(ValueError):
        stage_layers(2, (0, 3))


def test_stage_param_tables_partition_the_full_table():
    cfg = LlamaConfig.tiny(n_layers=4)
    full = ParamLayout(cfg)
    names = []
    for s in range(2):
        lay = ParamLayout(cfg, (s, 2))
        for n, (_, shape) in lay.entries.items():
            assert full.entries[n][1] == shape
            assert stage_of(cfg, n, 2) == s
        names += list(lay.entries)
    assert sorted(names) == sorted(full.entries)
    assert ParamLayout(cfg, (0, 2)).total + ParamLayout(cfg, (1, 2)).total == full.total


@pytest.mark.parametrize("p,m", [(2, 4), (4, 8), (8, 8)])
def test_fused_pipeline_streams_are_in_order_per_model_and_phase(p, m):
    """What the fused actor/critic executor relies on: for every (model, phase) the messages between two
    neighbouring devices are sent and received in the same order, the actor and the reversed critic meet every
    device exactly once per stage, and every device's instruction stream holds all of its tasks."""
    from rpeg_b200.parallel.fused_pp import logical_stage, uniform_schedule
    sched = uniform_schedule(p, {"actor": m, "critic": m})
    spec = {mm.name: mm for mm in sched.models}
    tasks = {t.task_id: t for t in sched.tasks}
    assert [logical_stage(spec["actor"], d) for d in range(p)] == list(range(p))
    assert [logical_stage(spec["critic"], d) for d in range(p)] == list(reversed(range(p)))
    assert all(len(o) == 4 * m for o in sched.device_order)
    for name, mm in spec.items():
        for phase in ("F", "B"):
            for s in range(p - 1):
                src_stage, dst_stage = (s, s + 1) if phase == "F" else (s + 1, s)
                sent = [tasks[t].microbatch for t in sched.device_order[mm.device_stage(src_stage)]
                        if tasks[t].model == name and tasks[t].phase == phase and tasks[t].stage == src_stage]
                got = [tasks[t].microbatch for t in sched.device_order[mm.device_stage(dst_stage)]
                       if tasks[t].model == name and tasks[t].phase == phase and tasks[t].stage == dst_stage]
                assert sent == got == list(range(m))


def test_version_and_slot_arithmetic_of_the_staleness_channels():
    """Iteration k consumes weight version max(0, k - 1 - tau) and produces version k; with tau + 2 slots the
    slot a producer writes is never one a consumer may still read."""
    from rpeg_b200.parallel.publish import consumed_version, slots_for
    from rpeg_b200.runtime.weight_versions import consumer_weight_version
    for tau in (0, 1, 2, 3):
        slots = slots_for(tau)
        assert slots == tau + 2
        for k in range(1, 12):
            v = consumed_version(k, tau)
            assert v == max(0, k - 1 - tau) == consumer_weight_version(k, tau)
            # while iteration k generates (reads slot v % slots) the trainers may be writing any version in
            # (v, k]: generation of k only starts after version v exists, training of k needs k's rollouts
            for w in range(v + 1, k + 1):
                assert w % slots != v % slots
