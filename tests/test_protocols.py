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


def test_guard_bytes_around_symmetric_buffers_catch_overruns(monkeypatch):
    """The allocator's canary logic, on host memory standing in for device memory: writes inside the buffer leave
    the guards alone; one byte past either end is reported with its side and offset."""
    import ctypes

    import torch

    from rpeg_b200.parallel import symm

    keep = {}

    class FakeLib:
        def rpeg_symm_alloc(self, nbytes, out):
            buf = (ctypes.c_ubyte * (int(nbytes) + 256))()                # cudaMalloc returns 256-byte aligned memory
            addr = (ctypes.addressof(buf) + 255) // 256 * 256
            keep[addr] = buf
            out._obj.value = addr
            return 0

        def rpeg_symm_free(self, ptr):
            keep.pop(int(ptr))
            return 0

    monkeypatch.setattr(symm, "lib", lambda: FakeLib())
    monkeypatch.setattr(symm, "wrap_device_memory",
                        lambda ptr, n, dev: torch.frombuffer((ctypes.c_ubyte * n).from_address(ptr), dtype=torch.uint8))
    buf = symm.SymmetricBuffer(1000, "cpu", zero=True)
    assert buf.nbytes == 1024 and buf.ptr % 256 == 0 and buf.ptr == buf.peer_ptrs[0]
    assert buf.bytes_view.data_ptr() == buf.ptr and int(buf.bytes_view.sum()) == 0
    buf.tensor(torch.float32)[:] = 1.0                                   # the whole usable range
    assert symm.check_canaries() >= 1 and buf.corrupted_guards() == []
    raw = (ctypes.c_ubyte * (buf.nbytes + 2 * symm.GUARD)).from_address(buf.ptr - symm.GUARD)
    raw[symm.GUARD + buf.nbytes + 3] = 0                                 # 4th byte past the end
    assert buf.corrupted_guards() == ["back+3"]
    with pytest.raises(symm.SymmetricMemoryCorruption, match=r"back\+3"):
        symm.check_canaries()
    raw[symm.GUARD + buf.nbytes + 3] = symm.CANARY
    raw[symm.GUARD - 1] = 7                                              # last byte before the start
    assert buf.corrupted_guards() == [f"front+{symm.GUARD - 1}"]
    raw[symm.GUARD - 1] = symm.CANARY
    buf.close()
    assert not keep and buf.ptr == 0 and buf.corrupted_guards() == []
    symm.check_canaries()


def test_checked_mode_validators_name_the_offending_index():
    """``ops/checked.py`` on CPU tensors: in-range arguments pass, every kind of stray index is reported with the
    kernel, the argument, the value and the allowed range."""
    import torch

    from rpeg_b200.ops import checked as C

    E = C.KernelArgumentError
    C.embed("k", torch.tensor([0, 5, 99], dtype=torch.int32), 100)
    with pytest.raises(E, match=r"k: ids\[1\] = 100 outside \[0, 100\)"):
        C.embed("k", torch.tensor([0, 100], dtype=torch.int32), 100)
    with pytest.raises(E, match=r"ids\[0\] = -1"):
        C.embed("k", torch.tensor([-1, 3], dtype=torch.int32), 100)
    cos = torch.zeros(128, 64)
    C.rope("k", torch.tensor([0, 127], dtype=torch.int32), 2, cos)
    with pytest.raises(E, match="pos"):
        C.rope("k", torch.tensor([0, 128], dtype=torch.int32), 2, cos)
    with pytest.raises(E, match="reads 3"):
        C.rope("k", torch.tensor([0, 1], dtype=torch.int32), 3, cos)
    # paged KV: pool of 6 pages (2 KV heads, head dim 128), 3 sequences x 4 pages
    kc = torch.zeros(6 * 2 * 64 * 128, dtype=torch.bfloat16)
    table = torch.tensor([[0, 1, 2, 3], [4, 5, 9, 9], [0, 0, 0, 0]], dtype=torch.int32)       # 9 = never used
    assert C.pool_pages(kc, 2, 128) == 6
    seq, pos = torch.tensor([0, 1, 1], dtype=torch.int32), torch.tensor([255, 0, 127], dtype=torch.int32)
    C.kv_append("k", 3, seq, pos, table, kc, 2, 128, torch.zeros(256, 64))
    with pytest.raises(E, match=r"page_table\[seq_id, pos // 64\]\[2\] = 9 outside \[0, 6\)"):
        C.kv_append("k", 3, seq, torch.tensor([255, 0, 128], dtype=torch.int32), table, kc, 2, 128)
    with pytest.raises(E, match="seq_id"):
        C.kv_append("k", 3, torch.tensor([0, 1, 3], dtype=torch.int32), pos, table, kc, 2, 128)
    with pytest.raises(E, match=r"pos\[0\] = 256 outside \[0, 256\)"):
        C.kv_append("k", 3, seq, torch.tensor([256, 0, 0], dtype=torch.int32), table, kc, 2, 128)
    with pytest.raises(E, match="rotary"):
        C.kv_append("k", 3, seq, pos, table, kc, 2, 128, torch.zeros(200, 64))
    C.kv_append("k", 2, seq, torch.tensor([255, 0, 999], dtype=torch.int32), table, kc, 2, 128)   # only the first 2 tokens count
    C.paged_attention("k", 3, torch.tensor([256, 128, 0], dtype=torch.int32), table, kc, 2, 128)
    with pytest.raises(E, match="pages in use"):
        C.paged_attention("k", 2, torch.tensor([256, 129], dtype=torch.int32), table, kc, 2, 128)  # reaches the stale entry
    with pytest.raises(E, match="seq_lens"):
        C.paged_attention("k", 1, torch.tensor([257], dtype=torch.int32), table, kc, 2, 128)
    with pytest.raises(E, match="4 rows"):
        C.paged_attention("k", 4, torch.tensor([1, 1, 1, 1], dtype=torch.int32), table, kc, 2, 128)
    C.packed_sequences("k", torch.tensor([0, 3, 3, 10], dtype=torch.int32), 10, 7)
    C.packed_sequences("k", torch.tensor([0, 3, 9], dtype=torch.int32), 10, 7)         # a padded token buffer
    for cu, n, mx in (([1, 3, 10], 10, 9), ([0, 5, 4, 10], 10, 9), ([0, 3, 11], 10, 9), ([0, 3, 10], 10, 6), ([0], 0, 1)):
        with pytest.raises(E):
            C.packed_sequences("k", torch.tensor(cu, dtype=torch.int32), n, mx)
    C.global_rows("k", torch.tensor([0, 7], dtype=torch.int64), 4, 2)
    with pytest.raises(E, match=r"global_idx\[1\] = 8"):
        C.global_rows("k", torch.tensor([0, 8], dtype=torch.int64), 4, 2)
    C.row_indices("k", torch.tensor([], dtype=torch.int32), 0)
    prev = C.set_enabled(True)
    try:
        assert C.active()                      # no capture is running on a machine without a GPU
    finally:
        C.set_enabled(prev)
    assert C.active() == prev


def test_flash_forward_pipeline_needs_one_completion_barrier_per_buffer():
    """The mbarrier pipeline of the flash attention forward kernel. With the P*V completion on ONE barrier that
    completes every tile and is consumed in order, a softmax warp can be two phases behind: the parity it waits for
    then names the running phase, which needs the warp's own next arrival (deadlock; on the GPU it ran into the
    bounded wait). Waiting directly on the wanted tile's parity of that single barrier passes too early instead. With
    one barrier per S/P buffer, as the kernel has it, every interleaving is clean for all rescale patterns."""
    from rpeg_b200.parallel.protocol_check import explore, flash_fwd_programs
    old = explore("in-order consumption of one barrier", flash_fwd_programs(5, (), pv_barriers=1, in_order_consume=True))
    assert old.finding is not None and old.finding.kind == "deadlock"
    early = explore("direct wait on one barrier", flash_fwd_programs(5, (3,), pv_barriers=1, in_order_consume=False))
    assert early.finding is not None and early.finding.kind == "race" and "P*V" in early.finding.message
    for n, resc in ((1, ()), (2, (1,)), (4, ()), (5, (1, 3)), (6, (2, 3, 5)), (7, (6,))):
        assert explore(f"{n} tiles", flash_fwd_programs(n, resc)).ok, (n, resc)


def test_one_exchange_allreduce_needs_two_slot_sets():
    """The all-reduce that pushes self-validating units and never acknowledges them: clean with the two slot sets the
    kernel alternates between, and the checker finds the overwritten units when there is only one."""
    for world, calls in ((2, 5), (3, 3)):
        assert pc.explore("two sets", pc.one_shot_allreduce_programs(world, calls)).ok
        bad = pc.explore("one set", pc.one_shot_allreduce_programs(world, calls, slot_sets=1))
        assert not bad.ok and bad.finding.kind == "race" and "units of call" in bad.finding.message
