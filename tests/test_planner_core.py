"""CPU tests of the analytical compiler: IR, unroll/lower passes, cost/memory models, scheduler."""
import math

import pytest

from rpeg_b200.analytic.cost import NodeCostModel
from rpeg_b200.analytic.hardware import Hardware, b200_nvswitch
from rpeg_b200.analytic.memory import MemoryPolicy, NodeMemoryModel, device_peaks, mem_feasible
from rpeg_b200.analytic.models import ModelSpec, ModelSuite
from rpeg_b200.analytic.workload import Workload
from rpeg_b200.core.types import (Allocation, Container, DeviceSpace, EdgeKind, Model, OperatorKind, Role, TemplateEdge,
                                  TemplateVertex, packing_geometry, rectangular_node_layouts)
from rpeg_b200.ir.plan import ExecutionPlan
from rpeg_b200.ir.rpeg import RPEG, IllFormedRPEG
from rpeg_b200.ir.templates import (build_AC_share_RPEG, build_DPO_RPEG, build_GRPO_RPEG, build_PPO_RPEG, build_rpeg)
from rpeg_b200.passes.lower import ExecNodeType, generation_phases, lower
from rpeg_b200.passes.unroll import publisher_selection, unroll
from rpeg_b200.schedule.scheduler import schedule
from rpeg_b200.search.evaluate import Configuration, evaluate_uncached, is_compatible, is_valid

SPEC = ModelSpec(32, 4096, 11008, 32000)
SUITE = ModelSuite({m: SPEC for m in Model})
WL = Workload(64, 1, 128, 512, ((0.5, 128), (0.85, 256), (1.0, 512)))
SPACE = DeviceSpace(1, 8, 4)


def example_hw() -> Hardware:
    ib = 1 / 12.5e9
    return Hardware(4.4e14, 103e9, 1.0e12, 78e-6, 1 / 220e9, 220e-6, ib, 220e-6, ib, 35e-6, 1 / 220e9, 180e-6, ib, 180e-6, ib,
                    gemm_m_half=240, decode_bw_eff=0.63, non_gemm_constant=0.12e-3, non_gemm_scaling=0.35e-3)


def spread_plan(rpeg, pi=(1, 1, 4)) -> ExecutionPlan:
    plan = ExecutionPlan()
    for i, v in enumerate(rpeg.vertices):
        plan.sigma[v.id], plan.pi[v.id], plan.mb[v.id] = Allocation((0, i, 0), (1, 1, 4)), pi, 1
    return plan


def test_param_count_and_geometry():
    assert SUITE.n_params(Model.ACTOR) == 32 * (4 * 4096 ** 2 + 2 * 4096 * 11008) + 32000 * 4096
    assert SUITE.n_params(Model.CRITIC) == SUITE.n_params(Model.ACTOR) + 4096
    assert packing_geometry(1, 1, 4, 4) == (4, 1)
    assert packing_geometry(2, 1, 2, 4) == (4, 1)
    assert packing_geometry(4, 2, 2, 4) == (4, 4)       # a replica fills a node, dp spans nodes
    assert packing_geometry(3, 1, 2, 4) is None          # fractional node
    assert packing_geometry(2, 8, 1, 4) == (4, 4)        # pipeline spans two nodes per replica
    assert packing_geometry(1, 1, 8, 4) is None          # TP group larger than a node
    assert rectangular_node_layouts(4, 2, 4) == [(1, 4), (2, 2)]
    assert is_compatible(Allocation((0, 2, 0), (1, 2, 4)), (4, 1, 2), SPACE)
    assert not is_compatible(Allocation((0, 7, 0), (1, 2, 4)), (4, 1, 2), SPACE)


@pytest.mark.parametrize("algo,nv,nd,npub", [("ppo", 6, 9, 2), ("grpo", 4, 4, 1), ("dpo", 3, 2, 1), ("ac_share", 5, 6, 2)])
def test_templates_are_well_formed(algo, nv, nd, npub):
    r = build_rpeg(algo, SUITE, WL)
    assert (len(r.vertices), len(r.data_edges), len(r.pub_edges)) == (nv, nd, npub)
    assert r.well_formed()
    assert all(t == 0 for t in r.tau.values())


def test_well_formedness_rejections():
    r = build_PPO_RPEG(SUITE, WL)
    with pytest.raises(IllFormedRPEG):
        RPEG(r.vertices, r.data_edges, r.pub_edges, r.containers, r.in_containers, (), {Model.ACTOR: 0}, r.trainable).well_formed()
    with pytest.raises(IllFormedRPEG):
        RPEG(r.vertices, r.data_edges, r.pub_edges[:1], r.containers, r.in_containers, (), r.tau, r.trainable).well_formed()
    with pytest.raises(IllFormedRPEG):
        RPEG(r.vertices, r.data_edges, r.pub_edges, r.containers, r.in_containers, (), {Model.ACTOR: -1, Model.CRITIC: 0}, r.trainable).well_formed()
    c = Container("x", 1, 2)
    a = TemplateVertex("a", OperatorKind(Role.INFERENCE, Model.REFERENCE, (c,), (c,)))
    b = TemplateVertex("b", OperatorKind(Role.INFERENCE, Model.REFERENCE, (c,), (c,)))
    with pytest.raises(IllFormedRPEG):
        RPEG((a, b), (TemplateEdge(a, b, c), TemplateEdge(b, a, c)), (), (c,), (), (), {}, set()).well_formed()


def test_unroll_publisher_selection_table():
    tau = {Model.ACTOR: 1, Model.CRITIC: 0}
    assert [publisher_selection(Model.ACTOR, tau, k) for k in range(5)] == [0, 0, 0, 1, 2]
    assert [publisher_selection(Model.CRITIC, tau, k) for k in range(5)] == [0, 0, 1, 2, 3]
    r = build_PPO_RPEG(SUITE, WL, tau=tau)
    u = unroll(r, 5)
    assert len(u.nodes) == 6 * 5 and len(u.data_edges) == 9 * 5
    # actor publishes only for k > 1, critic for k > 0
    assert len(u.pub_edges) == 3 + 4
    assert all(e.src.k < e.dst.k for e in u.pub_edges)
    pairs = {(e.src.id, e.dst.id) for e in u.pub_edges}
    assert ("t_pi@0", "g_pi@2") in pairs and ("t_V@3", "i_V@4") in pairs and ("t_pi@0", "g_pi@1") not in pairs


def test_generation_phases_from_quantiles():
    ph = generation_phases(WL)
    assert [(p.n_active, p.n_seqs, p.steps, p.t_start, p.is_prefill) for p in ph] == [
        (64, 32, 127, 0, True), (32, 22, 128, 127, False), (10, 10, 256, 255, False)]


def test_lower_splits_generation_and_inserts_comm():
    r = build_PPO_RPEG(SUITE, WL)
    low = lower(r, unroll(r, 2), spread_plan(r), SUITE, 2, workload=WL)
    ids = {n.id for n in low.nodes}
    assert {"g_pi@0:g0", "g_pi@0:g2", "i_ref@0:i1", "i_V@1:i2", "t_pi@1"} <= ids and "g_pi@0" not in ids
    kinds = [n.kind for n in low.nodes]
    assert kinds.count(ExecNodeType.RESHARD) == 0
    comm = [n for n in low.nodes if n.kind is ExecNodeType.COMM]
    # per step: 3 inference vertices x 3 phases from generation, 6 inference->train edges; plus 2 publications
    assert len(comm) == 2 * (9 + 6) + 2
    assert all(n.payload_in_bytes > 0 for n in comm)
    assert sorted(n.label for n in comm if n.label.startswith("W_")) == ["W_Pi", "W_V"]
    # colocated plan: no split, publication becomes an edge, nothing is transferred
    plan = ExecutionPlan()
    for v in r.vertices:
        plan.sigma[v.id], plan.pi[v.id], plan.mb[v.id] = Allocation((0, 0, 0), (1, 1, 4)), (1, 1, 4), 1
    low2 = lower(r, unroll(r, 2), plan, SUITE, 2, workload=WL)
    assert all(n.kind is ExecNodeType.OP for n in low2.nodes) and len(low2.nodes) == 12


def test_lower_reshard_and_fusion_composite():
    r = build_PPO_RPEG(SUITE, WL)
    plan = ExecutionPlan()
    box = Allocation((0, 0, 0), (1, 2, 4))
    for v in r.vertices:
        plan.sigma[v.id], plan.pi[v.id], plan.mb[v.id] = box, (4, 1, 2), 1
    for t in ("t_pi", "t_V"):
        plan.pi[t], plan.mb[t] = (1, 4, 2), 8
    low = lower(r, unroll(r, 2), plan, SUITE, 2, workload=WL, intra_stage_fusion=True)
    resh = [n for n in low.nodes if n.kind is ExecNodeType.RESHARD]
    # per step: g_pi -> t_pi and i_V -> t_V layout changes; across steps: both publications
    assert len(resh) == 2 * 2 + 2
    assert all(n.payload_in_bytes == SUITE.n_params(n.model) * 2 for n in resh)
    assert [c.id for c in low.composite_operators] == ["t_pi||V@0", "t_pi||V@1"]
    assert low.by_id()["t_pi@0"].fusion_group == "actor_critic_train@0"


def test_cost_and_schedule_match_reference_values():
    """Golden numbers produced by the reference's own analytical code (with its import-time
    defects repaired in a scratch copy) for the same inputs."""
    r = build_PPO_RPEG(SUITE, WL)
    cfg = Configuration(r, spread_plan(r), SPACE)
    score, trace, feasible = evaluate_uncached(cfg, SUITE, WL, example_hw(), 5)
    assert feasible and len(trace.start) == 153
    assert score == pytest.approx(2066.414637190287, rel=1e-12)
    assert trace.makespan() == pytest.approx(99.10886049397494, rel=1e-12)
    assert trace.utilization() == pytest.approx(0.19229326379208167, rel=1e-9)


def test_scheduler_respects_dependencies_and_devices():
    r = build_GRPO_RPEG(SUITE, Workload(64, 4, 128, 256))
    plan = ExecutionPlan()
    for i, v in enumerate(r.vertices):
        plan.sigma[v.id], plan.pi[v.id], plan.mb[v.id] = Allocation((0, i % 2, 0), (1, 1, 4)), (1, 1, 4), 1
    wl = Workload(64, 4, 128, 256)
    low = lower(r, unroll(r, 3), plan, SUITE, 3, workload=wl)
    tr = schedule(low, NodeCostModel(example_hw(), SUITE, wl), SPACE)
    for e in low.edges:
        assert tr.finish[e.src] <= tr.start[e.dst] + 1e-9
    busy = {}
    for n in low.nodes:
        for a in tr.reserved_allocations[n]:
            for d in a.coords():
                busy.setdefault(d, []).append((tr.start[n], tr.finish[n]))
    for spans in busy.values():
        spans.sort()
        assert all(a[1] <= b[0] + 1e-9 for a, b in zip(spans, spans[1:]))


def test_memory_model_terms():
    mm = NodeMemoryModel(example_hw(), SUITE, WL, optimizer_stage=2)
    r = build_PPO_RPEG(SUITE, WL)
    low = lower(r, unroll(r, 1), spread_plan(r, (1, 1, 4)), SUITE, 1, workload=WL)
    t = low.by_id()["t_pi@0"]
    layer = 4 * 4096 ** 2 + 2 * 4096 * 11008
    shard = math.ceil(32 * layer / 4) + 2 * 32000 * 4096
    assert mm.shard_params(t) == shard
    assert mm.weight_bytes(t) == 2 * shard and mm.optimizer_bytes(t) == 12 * shard and mm.gradient_bytes(t) == 2 * shard
    c = max(1, math.isqrt(32))
    per_token = math.ceil(32 / c) * 4096 + c * max(2 * 4096 + 6 * 4096 / 4, 2 * 4096 + 2 * 11008 / 4)
    assert mm.train_activation_bytes(t) == pytest.approx(2 * 64 * 640 * per_token)
    g = low.by_id()["g_pi@0:g0"]
    assert mm.kv_cache_bytes(g) == pytest.approx(2 * 2 * 64 * 640 * 32 * 4096 / 4)
    peaks = device_peaks(low, NodeMemoryModel.from_policy(example_hw(), SUITE, WL, MemoryPolicy(), trainable=frozenset(r.trainable)))
    assert len(peaks) == 24 and all(p > 0 for p in peaks.values())
    assert not mem_feasible(low, NodeMemoryModel(example_hw().with_updates(memory_per_gpu=1e9), SUITE, WL, trainable=frozenset(r.trainable)))


def test_nvswitch_fabric_cheaper_collectives_and_overlap():
    r = build_PPO_RPEG(SUITE, WL)
    low = lower(r, unroll(r, 1), spread_plan(r), SUITE, 1, workload=WL)
    node = low.by_id()["t_pi@0"]
    ring = NodeCostModel(b200_nvswitch().with_updates(fabric="ring"), SUITE, WL)
    sw = NodeCostModel(b200_nvswitch(), SUITE, WL)
    hidden = NodeCostModel(b200_nvswitch().with_updates(fused_overlap=0.8), SUITE, WL)
    assert sw.time_breakdown(node).intra_comm < ring.time_breakdown(node).intra_comm
    assert hidden.time_breakdown(node).intra_comm == pytest.approx(0.2 * sw.time_breakdown(node).intra_comm)
    assert hidden.time_breakdown(node).gemm == sw.time_breakdown(node).gemm


def test_engine_terms_of_the_cost_model():
    """The engine terms are off by default and each one moves the prediction the way the engine behaves."""
    r = build_PPO_RPEG(SUITE, WL)
    plan = ExecutionPlan()
    for v in r.vertices:                                       # colocated: generation and inference stay unsplit
        plan.sigma[v.id], plan.pi[v.id], plan.mb[v.id] = Allocation((0, 0, 0), (1, 1, 4)), (4, 1, 1), 1
    low = lower(r, unroll(r, 1), plan, SUITE, 1, workload=WL).by_id()
    train, inf, gen = low["t_pi@0"], low["i_ref@0"], low["g_pi@0"]
    base_hw = b200_nvswitch()
    base = NodeCostModel(base_hw, SUITE, WL)
    # gated MLP: the GEMM term grows by the parameter ratio (4 d^2 + 3 d f) / (4 d^2 + 2 d f), the attention part stays
    gated = NodeCostModel(base_hw.with_updates(ffn_matrices=3.0), SUITE, WL)
    d, f, seq = SPEC.d, SPEC.d_ff, WL.S + WL.T
    ratio = (4 * d * d + 3 * d * f + seq * d) / (4 * d * d + 2 * d * f + seq * d)
    assert gated.time_breakdown(inf).gemm / base.time_breakdown(inf).gemm == pytest.approx(ratio, rel=0.02)
    # sustained rate: compute-bound operators slow down by exactly the fraction
    sust = NodeCostModel(base_hw.with_updates(sustained_flops_fraction=0.8), SUITE, WL)
    assert sust.time_breakdown(train).gemm == pytest.approx(base.time_breakdown(train).gemm / 0.8)
    # attention at half the GEMM rate costs the attention FLOPs once more; elementwise time is linear in tokens
    att = NodeCostModel(base_hw.with_updates(attention_flops_eff=0.5), SUITE, WL)
    extra = att.time_breakdown(train).non_gemm - base.time_breakdown(train).non_gemm
    att_flops = 4 * WL.B * WL.K * seq * 2 * SPEC.L * seq * d
    assert extra == pytest.approx(att_flops / (4 * base_hw.flops_per_gpu))
    ew = NodeCostModel(base_hw.with_updates(elementwise_s_per_token_layer=1e-8), SUITE, WL)
    assert ew.time_breakdown(inf).non_gemm - base.time_breakdown(inf).non_gemm == pytest.approx(WL.B * WL.K * seq * SPEC.L / 4 * 1e-8)
    # generator limits: fewer rows decoding together -> the weights are streamed more often -> slower; a pool too small
    # for the batch acts like a slot limit
    t0 = base.time(gen)
    slots = NodeCostModel(base_hw.with_updates(gen_max_concurrency=4.0), SUITE, WL).time(gen)
    pool = NodeCostModel(base_hw.with_updates(gen_kv_budget_bytes=4.0 * 2 * d * 2 * SPEC.L * (WL.S + WL.T / 2)), SUITE, WL).time(gen)
    roomy = NodeCostModel(base_hw.with_updates(gen_max_concurrency=1e6, gen_kv_budget_bytes=1e15), SUITE, WL).time(gen)
    assert slots > 1.5 * t0 and roomy == pytest.approx(t0)
    if gen.phase_steps is None:
        assert pool == pytest.approx(slots, rel=1e-6)
    step = NodeCostModel(base_hw.with_updates(decode_step_overhead_s=1e-3), SUITE, WL).time(gen) - t0
    assert step > 0


def test_cost_model_with_expected_lengths():
    """With ``expected_lengths`` set, unsplit vertices are priced on the length quantiles: rows that stop early make
    generation, inference and training cheaper; shared prompt pages lower generation further; off by default."""
    import dataclasses
    wl = dataclasses.replace(WL, gen_quantiles=((0.5, WL.T // 4), (0.9, WL.T // 2), (1.0, WL.T)))
    r = build_PPO_RPEG(SUITE, wl)
    plan = ExecutionPlan()
    for v in r.vertices:
        plan.sigma[v.id], plan.pi[v.id], plan.mb[v.id] = Allocation((0, 0, 0), (1, 1, 4)), (4, 1, 1), 1
    low = lower(r, unroll(r, 1), plan, SUITE, 1, workload=wl).by_id()
    train, inf, gen = low["t_pi@0"], low["i_ref@0"], low["g_pi@0"]
    assert gen.n_active is None and inf.n_seqs is None               # colocated plan: not split by the quantiles
    hw = b200_nvswitch().with_updates(decode_step_overhead_s=1e-4)
    cap = NodeCostModel(hw, SUITE, wl)
    lens = NodeCostModel(hw.with_updates(expected_lengths=1.0), SUITE, wl)
    mean = 0.5 * wl.T / 8 + 0.4 * (wl.T / 4 + wl.T / 2) / 2 + 0.1 * (wl.T / 2 + wl.T) / 2
    assert lens._mean_len() == pytest.approx(mean) and cap._mean_len() == wl.T
    assert lens._seq_len(inf) == pytest.approx(wl.S + mean) and cap._seq_len(inf) == wl.S + wl.T
    for node in (train, inf, gen):
        assert lens.time(node) < cap.time(node)
    # the decode loop still runs to the longest row: generation shrinks by less than the token count does
    assert lens.time(gen) / cap.time(gen) > mean / wl.T * 0.5
    shared = NodeCostModel(hw.with_updates(expected_lengths=1.0, gen_shared_prompt_cost=0.5), SUITE, wl)
    if wl.K > 1:
        assert shared.time(gen) < lens.time(gen)
    else:
        assert shared.time(gen) == pytest.approx(lens.time(gen))
    # a generator with few slots decodes the rows in waves: slower, and never faster than the unlimited one
    few = NodeCostModel(hw.with_updates(expected_lengths=1.0, gen_max_concurrency=2.0), SUITE, wl)
    assert few.time(gen) > lens.time(gen)
    # without quantiles in the workload the switch changes nothing
    nq = dataclasses.replace(WL, gen_quantiles=None)
    r2 = build_PPO_RPEG(SUITE, nq)
    plain = lower(r2, unroll(r2, 1), plan, SUITE, 1, workload=nq).by_id()["g_pi@0"]
    assert NodeCostModel(hw.with_updates(expected_lengths=1.0), SUITE, nq).time(plain) == pytest.approx(NodeCostModel(hw, SUITE, nq).time(plain))


def test_validity_gate():
    r = build_PPO_RPEG(SUITE, WL)
    mm = NodeMemoryModel.from_policy(example_hw(), SUITE, WL, MemoryPolicy(), trainable=frozenset(r.trainable))
    good = Configuration(r, spread_plan(r), SPACE)
    assert is_valid(good, SUITE, WL, mm)
    bad = spread_plan(r)
    bad.mb["t_pi"] = 4                      # microbatches without a pipeline
    assert not is_valid(Configuration(r, bad, SPACE), SUITE, WL, mm)
    stale = build_PPO_RPEG(SUITE, WL, tau={Model.ACTOR: 1, Model.CRITIC: 0})
    colo = spread_plan(stale)
    colo.sigma["g_pi"] = colo.sigma["t_pi"]  # stale consumer must not share devices with its trainer
    assert not is_valid(Configuration(stale, colo, SPACE), SUITE, WL, mm)
