"""The device-side signalling protocols, checked over every interleaving of small instances on the host."""
import pytest

from rpeg_b200.parallel import protocol_check as pc
from rpeg_b200.parallel.publish import slots_for

W0 = {("w", r, s): 0 for r in range(3) for s in range(3)}


def test_every_protocol_is_clean_as_the_host_code_runs_it():
    results = pc.check_all()
    assert len(results) >= 12
    bad = [f"{r.name}: {r.finding}" for r in results if not r.ok]
    assert not bad, bad
    assert all(r.states > 10 for r in results)


def test_explorer_reports_races_torn_reads_and_deadlocks():
    # a reader that does not wait for the flag can see the old value, or the buffer half written
    writer = pc.bulk("buf", 1) + [("store", "flag", 1)]
    r = pc.explore("no wait", [writer, [("expect", "buf", 1, "reads early")]])
    assert not r.ok and r.finding.kind == "race" and "reads early" in r.finding.message
    assert pc.explore("with wait", [writer, [("wait", "flag", 1), ("expect", "buf", 1)]]).ok
    # flag raised before the data: the reader can pass the wait and still see the write in progress
    early = [("store", "flag", 1)] + pc.bulk("buf", 1)
    r = pc.explore("flag first", [early, [("wait", "flag", 1), ("expect", "buf", 1)]])
    assert not r.ok and ("being overwritten" in r.finding.message or "saw 0" in r.finding.message)
    # two ranks that each wait for the other's flag before setting their own never move
    r = pc.explore("cycle", [[("wait", "a", 1), ("store", "b", 1)], [("wait", "b", 1), ("store", "a", 1)]])
    assert not r.ok and r.finding.kind == "deadlock" and r.finding.trace == []
    # the trace ends with the offending read
    r = pc.explore("trace", [[("store", "x", 1), ("store", "x", 2)], [("expect", "x", 1)]])
    assert r.finding.trace[-1] == (1, ("expect", "x", 1))


@pytest.mark.parametrize("kwargs, what", [
    (dict(barrier_before_reduce=False), "reduces its shard"),          # peers' gradients not finished
    (dict(barrier_after_push=False), "reads shard"),                   # next forward before every shard has landed
    (dict(payload_slot_shared=True), "barrier payload"),               # a payload overwritten before a slow rank read it
])
def test_data_parallel_step_needs_each_of_its_barriers(kwargs, what):
    r = pc.explore("dp", pc.dp_step_programs(2, 2, **kwargs), W0)
    assert not r.ok and r.finding.kind == "race" and what in r.finding.message


def test_fused_linears_need_their_second_buffer_or_barrier():
    r = pc.explore("rs", pc.gemm_rs_programs(2, 3, buffers=1))
    assert not r.ok and "sums rank" in r.finding.message               # call e + 1 pushed over call e's partials
    r = pc.explore("ar", pc.gemm_rs_programs(2, 2, all_reduce=True, tail_barrier=False))
    assert not r.ok and "rows owned by rank" in r.finding.message      # output read before the peer's rows landed
    # all-gather + GEMM: with two operand buffers the arrival counters alone order the pushes (the barrier the host
    # issues is a second safeguard, not the only one)
    assert pc.explore("ag", pc.ag_gemm_programs(3, 3, barrier=False)).ok


@pytest.mark.parametrize("tau", [0, 1, 2])
def test_staleness_slot_count(tau):
    progs, init = pc.staleness_programs(tau, 6 + tau)
    assert pc.explore("default", progs, init).ok                       # slots_for(tau) copies, no acknowledgements
    assert slots_for(tau) >= tau + 1
    if tau > 0:
        progs, init = pc.staleness_programs(tau, 6 + tau, slots=tau)
        r = pc.explore("too few", progs, init)
        assert not r.ok and "being overwritten" in r.finding.message
