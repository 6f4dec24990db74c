"""Host-side model checker for the device-side signalling protocols.

The fused kernels and the peer-memory channels synchronise GPUs with a handful of primitives: release stores of
epoch / version words, arrival counters raised with system-scope reductions, bounded acquire waits, and bulk data
written into a peer's buffer before the word that announces it. Whether a protocol built from these is free of
races and deadlocks does not depend on the GPU, so it is checked here, exhaustively, on small instances: every
rank is a straight-line program of atomic steps (its stream order), a state is the vector of program counters plus
the contents of the shared words, and the checker walks EVERY interleaving of the ranks' steps. It reports

* a read that saw data of the wrong call / version, or data in the middle of being overwritten (a race),
* a state in which some rank waits and no rank can move (a deadlock),

with the interleaving that leads there. The programs below are the sequences the host code issues
(``parallel/tp.py``, ``parallel/dp.py``, ``parallel/publish.py`` with ``engine/async_rl.py``) and use the same
buffer-parity, call-count and slot arithmetic; each has switches that remove one ingredient (a barrier, the second
buffer, a slot) so that tests can show the checker finds the race the ingredient prevents.

The reference has no device-side protocols of its own; its closest check is the blocking point-to-point rendezvous
simulation that proves its fused pipeline schedules deadlock free (RPEG/runtime/fused_pipeline.py:626-745) and the
resource-overlap rule of its trace verifier (RPEG/runtime/verification.py:860-875).

``python -m rpeg_b200.parallel.protocol_check`` runs every model and prints one line per model.
"""
from __future__ import annotations

import sys
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

Instr = Tuple
Program = List[Instr]

# Instructions (loc is any hashable name of a shared word or buffer region):
#   ("store", loc, value)          one atomic store (a release store of a flag, or a small payload)
#   ("begin", loc, value)          first byte of a bulk write: the region is torn until the matching "end"
#   ("end", loc, value)            last byte of the bulk write has landed: the region holds `value`
#   ("add", loc, n)                atomic add (arrival counter)
#   ("wait", loc, minimum)         blocks while the word is below `minimum` (an acquire spin; bounded on the device)
#   ("expect", loc, value, what)   a read that must see exactly `value`; anything else is reported as a race
#   ("pwait", loc, parity)         mbarrier.try_wait.parity: the word counts the barrier's completed phases; the wait
#                                  passes while the CURRENT phase's parity differs from `parity`, i.e. it cannot tell a
#                                  phase that completed from one that completed two phases ago
#   ("check", loc, minimum, what)  an assertion: the word must have reached `minimum` (reported as a race otherwise)
TORN = "torn"


@dataclass
class Finding:
    kind: str                       # "race" or "deadlock"
    message: str
    trace: List[Tuple[int, Instr]]  # (rank, instruction) in execution order

    def __str__(self) -> str:
        tail = "; ".join(f"r{r}:{' '.join(map(str, i[:3]))}" for r, i in self.trace[-8:])
        return f"{self.kind}: {self.message} after {len(self.trace)} steps (... {tail})"


@dataclass
class Result:
    name: str
    states: int
    finding: Optional[Finding]

    @property
    def ok(self) -> bool:
        return self.finding is None


def explore(name: str, programs: Sequence[Program], initial: Optional[Dict[Hashable, object]] = None,
            max_states: int = 2_000_000) -> Result:
    """Walk every interleaving of ``programs`` (depth first, visited states remembered)."""
    n = len(programs)
    mem0 = dict(initial or {})
    start = (tuple([0] * n), tuple(sorted(mem0.items(), key=repr)))
    parent: Dict[tuple, Optional[Tuple[tuple, int, Instr]]] = {start: None}
    stack = [start]

    def trace_of(state, last: Optional[Tuple[int, Instr]] = None) -> List[Tuple[int, Instr]]:
        out: List[Tuple[int, Instr]] = [] if last is None else [last]
        while parent[state] is not None:
            state, r, ins = parent[state]
            out.append((r, ins))
        out.reverse()
        return out

    while stack:
        state = stack.pop()
        pcs, items = state
        mem = dict(items)
        moved = False
        for r in range(n):
            if pcs[r] >= len(programs[r]):
                continue
            ins = programs[r][pcs[r]]
            op, loc = ins[0], ins[1]
            cur = mem.get(loc, 0)
            new = None                      # None: memory unchanged
            if op == "wait":
                if cur == TORN or not isinstance(cur, int) or cur < ins[2]:
                    continue
            elif op == "pwait":
                if (int(cur) & 1) == (int(ins[2]) & 1):
                    continue
            elif op == "check":
                if not isinstance(cur, int) or cur < ins[2]:
                    what = ins[3] if len(ins) > 3 else "assertion"
                    return Result(name, len(parent), Finding("race", f"rank {r} {what}: {loc} should have reached {ins[2]}, is {cur!r}",
                                                            trace_of(state, (r, ins))))
            elif op == "expect":
                if cur != ins[2]:
                    what = ins[3] if len(ins) > 3 else "read"
                    seen = "a buffer that is being overwritten" if isinstance(cur, tuple) and cur and cur[0] == TORN else repr(cur)
                    return Result(name, len(parent), Finding("race", f"rank {r} {what}: {loc} should hold {ins[2]!r}, saw {seen}",
                                                            trace_of(state, (r, ins))))
            elif op == "store" or op == "end":
                new = ins[2]
            elif op == "begin":
                new = (TORN, ins[2])
            elif op == "add":
                new = (cur if isinstance(cur, int) else 0) + ins[2]
            else:
                raise ValueError(f"unknown instruction {ins!r}")
            moved = True
            if new is None:
                nitems = items
            else:
                m2 = dict(mem)
                m2[loc] = new
                nitems = tuple(sorted(m2.items(), key=repr))
            nxt = (pcs[:r] + (pcs[r] + 1,) + pcs[r + 1:], nitems)
            if nxt not in parent:
                parent[nxt] = (state, r, ins)
                stack.append(nxt)
                if len(parent) > max_states:
                    raise RuntimeError(f"{name}: more than {max_states} states; check a smaller instance")
        if not moved and any(pcs[r] < len(programs[r]) for r in range(n)):
            stuck = {r: programs[r][pcs[r]] for r in range(n) if pcs[r] < len(programs[r])}
            return Result(name, len(parent), Finding("deadlock", f"no rank can move; waiting: {stuck}", trace_of(state)))
    return Result(name, len(parent), None)


# ---------------------------------------------------------------------------------------------- building blocks
def bulk(loc, value) -> Program:
    return [("begin", loc, value), ("end", loc, value)]


def flag_barrier(pad: str, rank: int, world: int, slot: int, epoch: int, payload=None) -> Program:
    """``flag_barrier_kernel``: thread t writes the optional payload, then the epoch, into rank t's pad (release),
    then waits for rank t's word in its own pad, then reads rank t's payload."""
    prog: Program = []
    for t in range(world):
        if payload is not None:
            prog.append(("store", (pad, "payload", t, slot, rank), payload))
        prog.append(("store", (pad, "flag", t, slot, rank), epoch))
    for t in range(world):
        prog.append(("wait", (pad, "flag", rank, slot, t), epoch))
    if payload is not None:
        for t in range(world):
            prog.append(("expect", (pad, "payload", rank, slot, t), payload, f"reads rank {t}'s barrier payload"))
    return prog


# ---------------------------------------------------------------------------------------------- the protocols
def dp_step_programs(world: int, steps: int, *, barrier_before_reduce: bool = True, barrier_after_push: bool = True,
                     payload_slot_shared: bool = False) -> List[Program]:
    """The fused data-parallel optimizer step (``DPContext.fused_adam_step``): backward writes this rank's
    gradient buffer and reads its weights; barrier 0; every rank reduces ITS shard from all ranks' gradient buffers
    (loads from peer memory); barrier 1 carries the partial squared norms; Adam on the shard, result pushed into
    every rank's weights; barrier 2. ``payload_slot_shared`` runs barrier 2 on barrier 1's slot with a payload of
    its own, which is the misuse the separate slots avoid."""
    progs: List[Program] = []
    for r in range(world):
        p: Program = []
        for k in range(1, steps + 1):
            for s in range(world):
                p.append(("expect", ("w", r, s), k - 1, f"forward of step {k} reads shard {s} of its weights"))
            p += bulk(("g", r), k)
            if barrier_before_reduce:
                p += flag_barrier("pad", r, world, 0, k)
            for q in range(world):
                p.append(("expect", ("g", q), k, f"reduces its shard of rank {q}'s gradients in step {k}"))
            p += flag_barrier("pad", r, world, 1, 2 * k - 1 if payload_slot_shared else k, payload=("norm", k))
            for q in range(world):
                p += bulk(("w", q, r), k)
            if barrier_after_push:
                if payload_slot_shared:
                    p += flag_barrier("pad", r, world, 1, 2 * k, payload=("landed", k))
                else:
                    p += flag_barrier("pad", r, world, 2, k)
        progs.append(p)
    return progs


def gemm_rs_programs(world: int, calls: int, *, buffers: int = 2, all_reduce: bool = False, tail_barrier: bool = True) -> List[Program]:
    """Row-parallel linear (``RowParallelLinear.forward`` + ``csrc/gemm_rs.cu``): call ``e`` uses buffer set
    ``e % buffers``; every rank pushes its partial of every owner's rows into the owner's staging area and raises
    the owner's arrival counter; the owner waits for ``(uses of this buffer set) * world`` arrivals, sums the
    partials and writes the result (all-reduce: into every rank's output, followed by a flag barrier so that no
    rank reads its output before every owner's rows have landed); the next kernel on the stream reads the output."""
    progs: List[Program] = []
    for r in range(world):
        p: Program = []
        for e in range(1, calls + 1):
            b = e % buffers
            uses = (e + buffers - 1) // buffers if buffers == 2 else e
            for q in range(world):
                p += bulk(("stage", q, b, r), e)
                p.append(("add", ("arrived", q, b), 1))
            p.append(("wait", ("arrived", r, b), uses * world))
            for s in range(world):
                p.append(("expect", ("stage", r, b, s), e, f"sums rank {s}'s partial in call {e}"))
            if all_reduce:
                for q in range(world):
                    p += bulk(("out", q, b, r), e)
                if tail_barrier:
                    p += flag_barrier("pad", r, world, 0, e)
                for s in range(world):
                    p.append(("expect", ("out", r, b, s), e, f"consumer of call {e} reads rows owned by rank {s}"))
            else:
                p += bulk(("out", r, b, r), e)
                p.append(("expect", ("out", r, b, r), e, f"consumer of call {e} reads its rows"))
        progs.append(p)
    return progs


def ag_gemm_programs(world: int, calls: int, *, barrier: bool = True) -> List[Program]:
    """Column-parallel linear (``ColumnParallelLinear.forward`` + ``csrc/ag_gemm.cu``): the caller writes its rows
    into its own copy of X (buffer ``e % 2``); a flag barrier; the kernel's copy warps push the rows into every
    peer's X and raise the peer's ready counter; its producer warp waits for ``uses * (world - 1)`` arrivals and the
    tensor-core tiles read all rows. The barrier keeps a fast rank from pushing call ``e``'s rows into a buffer that
    a slow peer still reads for call ``e - 2``."""
    progs: List[Program] = []
    for r in range(world):
        p: Program = []
        for e in range(1, calls + 1):
            b = e % 2
            uses = (e + 1) // 2
            p += bulk(("x", r, b, r), e)
            if barrier:
                p += flag_barrier("pad", r, world, 0, e)
            for q in range(world):
                if q != r:
                    p += bulk(("x", q, b, r), e)
                    p.append(("add", ("ready", q, b), 1))
            p.append(("wait", ("ready", r, b), uses * (world - 1)))
            for s in range(world):
                p.append(("expect", ("x", r, b, s), e, f"GEMM of call {e} reads rank {s}'s rows"))
        progs.append(p)
    return progs


def staleness_programs(tau: int, steps: int, *, slots: Optional[int] = None, n_gen: int = 1, n_train: int = 1) -> Tuple[List[Program], Dict]:
    """Disaggregated training with bounded staleness (``AsyncGRPO``): generation rank(s) read weight version
    ``max(0, k - 1 - tau)`` for the whole of iteration ``k`` and then push the rollouts of ``k`` to every trainer;
    trainers wait for the rollouts of ``k`` from every generator, train, and push version ``k`` of their weight share
    into slot ``k % slots`` of every generator. No acknowledgements: safety rests on the slot count alone."""
    from .publish import consumed_version, slots_for
    n_slots = slots_for(tau) if slots is None else slots
    progs: List[Program] = []
    for gi in range(n_gen):
        p: Program = []
        for k in range(1, steps + 1):
            v = consumed_version(k, tau)
            s = v % n_slots
            for t in range(n_train):
                if v > 0:
                    p.append(("wait", ("wver", gi, s, t), v))
            for phase in ("first", "last"):
                for t in range(n_train):
                    p.append(("expect", ("wts", gi, s, t), v, f"generator {gi}, iteration {k}, {phase} decode step reads trainer {t}'s share"))
            for t in range(n_train):
                p += bulk(("rows", t, k % n_slots, gi), k)
                p.append(("store", ("rver", t, k % n_slots, gi), k))
        progs.append(p)
    for t in range(n_train):
        p = []
        for k in range(1, steps + 1):
            s = k % n_slots
            for gi in range(n_gen):
                p.append(("wait", ("rver", t, s, gi), k))
            for phase in ("reference pass", "policy step"):
                for gi in range(n_gen):
                    p.append(("expect", ("rows", t, s, gi), k, f"trainer {t}, step {k}, {phase} reads generator {gi}'s rows"))
            for gi in range(n_gen):
                p += bulk(("wts", gi, s, t), k)
                p.append(("store", ("wver", gi, s, t), k))
        progs.append(p)
    initial = {("wts", gi, 0, t): 0 for gi in range(n_gen) for t in range(n_train)}
    return progs, initial


# ---------------------------------------------------------------------------------------------- the suite
def flash_fwd_programs(n_tiles: int, rescale: Sequence[int] = (), *, pv_barriers: int = 2, in_order_consume: bool = False) -> List[Program]:
    """The mbarrier pipeline of ``flash_attn_fwd_kernel`` (csrc/flash_attn.cu) for one CTA and ``n_tiles`` KV tiles, as
    three agents: the MMA-issuing thread, the tensor pipe (completes the issued MMAs in issue order, each at an
    arbitrary later time, and performs their commits) and one softmax warp. ``rescale``: the tiles at which the warp
    rescales O and therefore waits for the previous P*V product. Words count completed phases of a barrier.

    ``pv_barriers = 2``: P*V of tile j commits to ``pv_done[j & 1]`` and the warp waits on the wanted tile's barrier
    with parity ``(j >> 1) & 1`` (the kernel as it is). ``pv_barriers = 1, in_order_consume = True``: one barrier that
    completes every tile, consumed in order with the oldest outstanding completion waited for at the top of each
    iteration. That version deadlocks: P*V of tile j-1 may complete before the warp tests for tile j-2, the parity
    then names the running phase, and that phase cannot end without the warp's own next P."""
    pv = (lambda j: ("pv_done", j & 1)) if pv_barriers == 2 else (lambda j: ("pv_done", 0))
    pv_par = (lambda j: (j >> 1) & 1) if pv_barriers == 2 else (lambda j: j & 1)
    mma: Program = [("add", "issued", 1)]                                    # QK_0
    pipe: Program = [("wait", "issued", 1), ("add", ("s_full", 0), 1)]
    n_issued = 1
    for j in range(n_tiles):
        if j + 1 < n_tiles:
            mma.append(("add", "issued", 1))                                 # QK_{j+1} under the softmax of tile j
            n_issued += 1
            pipe += [("wait", "issued", n_issued), ("add", ("s_full", (j + 1) & 1), 1)]
        mma += [("pwait", ("p_full", j & 1), (j >> 1) & 1), ("add", "issued", 1)]   # P_j delivered -> P*V_j
        n_issued += 1
        pipe += [("wait", "issued", n_issued), ("add", "pv_count", 1), ("add", pv(j), 1)]
    warp: Program = []
    seen = 0
    for j in range(n_tiles):
        warp.append(("pwait", ("s_full", j & 1), (j >> 1) & 1))
        if in_order_consume:
            while seen <= j - 2:
                warp.append(("pwait", pv(seen), pv_par(seen)))
                seen += 1
        if j in rescale and j > 0:
            if in_order_consume:
                while seen <= j - 1:
                    warp.append(("pwait", pv(seen), pv_par(seen)))
                    seen += 1
            else:
                warp.append(("pwait", pv(j - 1), pv_par(j - 1)))
            warp.append(("check", "pv_count", j, f"rescales O at tile {j} before P*V of tile {j - 1} has landed"))
        warp.append(("add", ("p_full", j & 1), 1))
    if in_order_consume:
        while seen <= n_tiles - 1:
            warp.append(("pwait", pv(seen), pv_par(seen)))
            seen += 1
    else:
        warp.append(("pwait", pv(n_tiles - 1), pv_par(n_tiles - 1)))
    warp.append(("check", "pv_count", n_tiles, "reads O before the last P*V has landed"))
    return [mma, pipe, warp]


def one_shot_allreduce_programs(world: int, calls: int, *, slot_sets: int = 2) -> List[Program]:
    """The one-exchange all-reduce of the tensor-parallel decode step (``csrc/tp_decode.cu``,
    ``tp_allreduce_rmsnorm_ll_kernel``): in call k every rank stores its units {data, k} into its own slot of set
    ``k % slot_sets`` in EVERY rank's region, then polls the slots of all senders in its own region until their units carry
    k, and reduces them. No flag follows the data and nothing is acknowledged: what keeps a sender from overwriting units
    that a slow receiver has not read yet is only that it cannot finish call k + 1 before that receiver has sent its own
    units of call k + 1, i.e. has finished reading call k. Two slot sets are therefore enough, one is not."""
    progs: List[Program] = []
    for r in range(world):
        p: Program = []
        for k in range(1, calls + 1):
            s = k % slot_sets
            for t in range(world):
                p.append(("store", ("ll", t, s, r), k))                 # a unit is one atomic 8-byte store
            for sender in range(world):
                p.append(("wait", ("ll", r, s, sender), k))
                p.append(("expect", ("ll", r, s, sender), k, f"reduces rank {sender}'s units of call {k}"))
        progs.append(p)
    return progs


def check_all(verbose: bool = False) -> List[Result]:
    """Every protocol as the host code runs it; all must come out clean."""
    out: List[Result] = []
    w0 = {("w", r, s): 0 for r in range(3) for s in range(3)}
    out.append(explore("dp step, 2 ranks x 3 steps", dp_step_programs(2, 3), w0))
    out.append(explore("dp step, 3 ranks x 2 steps", dp_step_programs(3, 2), w0))
    out.append(explore("gemm + reduce-scatter, 2 ranks x 4 calls", gemm_rs_programs(2, 4)))
    out.append(explore("gemm + reduce-scatter, 3 ranks x 3 calls", gemm_rs_programs(3, 3)))
    out.append(explore("gemm + all-reduce, 2 ranks x 4 calls", gemm_rs_programs(2, 4, all_reduce=True)))
    out.append(explore("all-gather + gemm, 2 ranks x 4 calls", ag_gemm_programs(2, 4)))
    out.append(explore("all-gather + gemm, 3 ranks x 3 calls", ag_gemm_programs(3, 3)))
    out.append(explore("one-exchange all-reduce, 2 ranks x 5 calls", one_shot_allreduce_programs(2, 5)))
    out.append(explore("one-exchange all-reduce, 3 ranks x 3 calls", one_shot_allreduce_programs(3, 3)))
    for tau in (0, 1, 2):
        progs, init = staleness_programs(tau, 5 + tau)
        out.append(explore(f"staleness {tau}, 1 generator + 1 trainer", progs, init))
    progs, init = staleness_programs(1, 4, n_gen=2, n_train=1)
    out.append(explore("staleness 1, 2 generators + 1 trainer", progs, init))
    progs, init = staleness_programs(1, 4, n_gen=1, n_train=2)
    out.append(explore("staleness 1, 1 generator + 2 trainers", progs, init))
    import itertools
    for n in (1, 2, 3, 5, 6):
        for k in range(0, min(n, 3)):
            for resc in itertools.combinations(range(1, n), k):
                out.append(explore(f"flash forward pipeline, {n} tiles, rescale at {list(resc)}", flash_fwd_programs(n, resc)))
    if verbose:
        for r in out:
            print(f"{'ok  ' if r.ok else 'FAIL'} {r.name}: {r.states} states" + ("" if r.ok else f" -- {r.finding}"))
    return out


def main(argv: Optional[List[str]] = None) -> int:
    results = check_all(verbose=True)
    return 0 if all(r.ok for r in results) else 1


if __name__ == "__main__":
    sys.exit(main())
