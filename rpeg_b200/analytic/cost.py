"""Analytical time model of executable nodes (OP, COMM, RESHARD).

The formulas are the reference's (RPEG/model/cost.py:34-686), restated around a small ``_Shape``
helper so each term reads like its definition:

OP time   = [ W / (F_eff * P) ] * (m + pp - 1)/m  +  t_intra_comm  +  t_non_gemm
            (+ 18 B/param optimizer traffic for TRAIN), times the per-role scale.
  W       work FLOPs of the role (prefill+decode for GEN, forward for INF, 3x or 4x forward for
          TRAIN depending on activation checkpointing),
  F_eff   roofline: ``F * eta`` above the ridge ``F/BW``, else ``intensity * BW``; ``eta`` is the
          GEMM saturation ``M/(M+M_half)`` (times a TP narrowing term); generation mixes a prefill
          and a decode regime with separate byte streams (weights, KV, activations),
  P       dp * pp * tp devices, m effective microbatch count.
COMM      alpha + payload / min(|src|, |dst|) * beta on the point-to-point tier of the two boxes.
RESHARD   all-to-all of payload / P on the collective tier.

With ``Hardware.fabric == "nvswitch"`` intra-node collectives use switch formulas (one hop,
in-switch reduction) and ``fused_overlap`` hides that fraction of TP/DP collectives behind math,
which is how the fused GEMM+collective and reduce-scatter+Adam kernels enter the plan search.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import NamedTuple, Tuple

from ..core.types import Allocation, Collective, Model, Role
from ..passes.lower import ExecNode, ExecNodeType
from .hardware import Hardware
from .models import ModelSuite
from .workload import Workload


class OpTimeBreakdown(NamedTuple):
    gemm: float
    bubble: float
    intra_comm: float
    non_gemm: float
    optimizer_step: float


@dataclass(frozen=True)
class _Shape:
    L: int
    d: int
    f: int
    V: int
    sb: int
    ffn: float = 2.0     # matrices of d x d_ff in the MLP (hardware.ffn_matrices)

    @property
    def layer_params(self) -> float:
        if self.ffn == 2.0:
            return 4 * self.d * self.d + 2 * self.d * self.f
        return 4 * self.d * self.d + self.ffn * self.d * self.f

    def layer_flops_per_token(self, ctx: float) -> float:
        """FLOPs / 2 of one layer for one token that attends to ``ctx`` positions."""
        return self.layer_params + ctx * self.d

    @property
    def params(self) -> int:
        return self.L * self.layer_params + self.V * self.d


_HEAD_FLOPS = {  # per-token head cost / 2, as a function of (V, d)
    Model.ACTOR: lambda V, d: V * d, Model.REFERENCE: lambda V, d: V * d,
    Model.CRITIC: lambda V, d: d, Model.AC_SHARE: lambda V, d: d,
}


@dataclass(frozen=True)
class NodeCostModel:
    hw: Hardware
    suite: ModelSuite
    workload: Workload
    optimizer_stage: int = 2
    activation_checkpointing: float = True      # True / False, or the FRACTION of the layers whose forward pass runs a second time

    def __post_init__(self):
        if self.optimizer_stage not in (0, 1, 2):
            raise ValueError("optimizer_stage must be 0, 1, or 2")
        for name in ("op_generation_scale", "op_inference_scale", "op_training_scale", "weight_comm_scale", "reshard_scale"):
            v = float(getattr(self.hw, name))
            if not math.isfinite(v) or v <= 0.0:
                raise ValueError(f"hardware.{name} must be finite and > 0")
        o = float(self.hw.activation_comm_overhead_s)
        if not math.isfinite(o) or o < 0.0:
            raise ValueError("hardware.activation_comm_overhead_s must be finite and >= 0")

    # ------------------------------------------------------------------ public
    def time(self, node: ExecNode) -> float:
        if node.kind is ExecNodeType.OP:
            return sum(self.time_breakdown(node))
        if node.kind is ExecNodeType.COMM:
            return self._comm_time(node)
        if node.kind is ExecNodeType.RESHARD:
            return self._reshard_time(node)
        raise ValueError(f"unknown node kind {node.kind}")

    def time_breakdown(self, node: ExecNode) -> OpTimeBreakdown:
        if node.kind is not ExecNodeType.OP:
            raise ValueError("time_breakdown is only valid for OP nodes")
        role = node.role
        pd, pp, pt = node.pi
        m = self._effective_mb(node)
        if role is Role.GENERATION and node.n_active is None and self._length_bins() is not None:
            gemm = self._generation_time_by_lengths(node)
        else:
            gemm = self._work(node) / (self._effective_flops(node) * pd * pp * pt)
        bubble = gemm * (pp - 1) / m
        opt = 0.0
        if role is Role.TRAINING:
            dp_shards = pd if self.optimizer_stage >= 1 else 1
            opt = self._shape(node.model).params / (dp_shards * pp * pt) * 18 / self.hw.memory_bandwidth
        scale = {Role.GENERATION: self.hw.op_generation_scale, Role.INFERENCE: self.hw.op_inference_scale,
                 Role.TRAINING: self.hw.op_training_scale}.get(role, 1.0)
        parts = (gemm, bubble, self._intra_comm(node), self._non_gemm(node) + self._engine_terms(node), opt)
        return OpTimeBreakdown(*(p * scale for p in parts))

    # ------------------------------------------------------------------ batch geometry
    def _shape(self, model: Model) -> _Shape:
        s = self.suite.specs[model]
        return _Shape(s.L, s.d, s.d_ff, s.V, s.dtype_bytes, float(self.hw.ffn_matrices))

    def _effective_batch(self, node: ExecNode) -> float:
        if node.n_active is not None:
            return node.n_active
        if node.n_seqs is not None:
            return node.n_seqs
        return self.workload.B * self.workload.K

    def _effective_mb(self, node: ExecNode) -> int:
        return max(1, min(node.mb, int(self._effective_batch(node)) // max(1, node.pi[0])))

    def _b_local(self, node: ExecNode) -> float:
        return self._effective_batch(node) / (node.pi[0] * self._effective_mb(node))

    # ------------------------------------------------------------------ work
    def _work(self, node: ExecNode) -> float:
        role, model = node.role, node.model
        sh = self._shape(model)
        w = self.workload
        BK, S, T = w.B * w.K, w.S, w.T
        if role is Role.GENERATION:
            prefill_row = S * 2 * sh.L * sh.layer_flops_per_token(S) + 2 * sh.V * sh.d
            if node.n_active is not None:
                n, steps = node.n_active, node.phase_steps
                past = S + node.phase_t_start + steps / 2
                work = n * (2 * steps * sh.L * sh.layer_flops_per_token(past) + 2 * steps * sh.V * sh.d)
                return work + (n * prefill_row if node.is_prefill_phase else 0)
            decode_row = 2 * (T - 1) * sh.L * sh.layer_flops_per_token(S + T / 2) + 2 * (T - 1) * sh.V * sh.d
            return BK * (prefill_row + decode_row)
        seq = self._seq_len(node)
        trunk = 2 * sh.L * sh.layer_flops_per_token(seq)
        if role is Role.INFERENCE:
            n = node.n_seqs if node.n_seqs is not None else BK
            if model is Model.REWARD:
                return n * seq * trunk + n * 2 * sh.d
            return n * seq * (trunk + 2 * _HEAD_FLOPS[model](sh.V, sh.d))
        if role is Role.TRAINING:
            mult = 3 + float(self.activation_checkpointing)
            head = {Model.ACTOR: 2 * sh.V * sh.d, Model.CRITIC: 2 * sh.d, Model.AC_SHARE: 2 * sh.V * sh.d + 2 * sh.d}
            if model in head:
                return mult * BK * seq * (trunk + head[model])
        raise ValueError(f"no work model for role={role} model={model}")

    # ------------------------------------------------------------------ roofline
    def _effective_flops(self, node: ExecNode) -> float:
        if node.role is Role.GENERATION:
            return self._generation_flops(node)
        hw, sh = self.hw, self._shape(node.model)
        pd, pp, pt = node.pi
        seq = self._seq_len(node)
        b = self._b_local(node)
        Lpp = sh.L / pp
        flops = b * seq * (2 * Lpp / pt) * sh.layer_flops_per_token(seq)
        nbytes = Lpp / pt * sh.layer_params * sh.sb + 2 * b * seq * sh.d * Lpp * sh.sb
        intensity = flops / nbytes if nbytes > 0 else float("inf")
        if intensity >= hw.flops_per_gpu / hw.memory_bandwidth:
            return hw.flops_per_gpu * hw.sustained_flops_fraction * self._gemm_efficiency(node, b * seq)
        return intensity * hw.memory_bandwidth

    def _length_bins(self):
        """``[(row fraction, first step, last step), ...]`` of the workload's length quantiles (rows of a bin stop
        uniformly inside it), or ``None`` when lengths are not to be used."""
        q = self.workload.gen_quantiles
        if not (self.hw.expected_lengths > 0 and q):
            return None
        bins, prev_f, prev_t = [], 0.0, 0
        for f, t in q:
            if f > prev_f:
                bins.append((float(f) - prev_f, int(prev_t), int(t)))
            prev_f, prev_t = float(f), int(t)
        return bins or None

    def _seq_len(self, node: ExecNode) -> float:
        """Tokens per row of an inference / training vertex: prompt + cap, or prompt + expected response length when
        the length quantiles are in use and the vertex is not already split by them."""
        if node.n_seqs is None and self._length_bins() is not None:
            return self.workload.S + self._mean_len()
        return float(self.workload.S + self.workload.T)

    def _mean_len(self) -> float:
        """Expected response length under the quantiles (``T`` without them)."""
        bins = self._length_bins()
        if bins is None:
            return float(self.workload.T)
        return sum(frac * (a + b) / 2.0 for frac, a, b in bins)

    def _generation_time_by_lengths(self, node: ExecNode) -> float:
        """Seconds of an unsplit generation vertex when rows stop at their own length: the decode loop runs until
        the longest row ends, the number of live rows falls along the length distribution (rows beyond the
        generator's concurrency wait and are decoded later), every step streams the weights once and the K/V of the
        live rows (a shared prompt token at ``gen_shared_prompt_cost`` of a private one)."""
        hw, sh, w = self.hw, self._shape(node.model), self.workload
        pd, pp, pt = node.pi
        Lpp = sh.L / pp
        rows = self._b_local(node) * self._effective_mb(node)           # rows of one replica
        bw = hw.memory_bandwidth
        w_bytes = Lpp / pt * sh.layer_params * sh.sb
        e_w = hw.decode_bw_eff
        e_kv = min(1.0, 3.5 * e_w)
        kv_tok = 2 * (sh.d / pt) * sh.sb * Lpp                          # K/V bytes of one cached token on one GPU
        share = hw.gen_shared_prompt_cost if (hw.gen_shared_prompt_cost < 1.0 and w.K > 1) else 1.0
        prompt_rows = rows / w.K if share < 1.0 else rows
        # prefill (once per prompt when the samples share it)
        m_half = hw.gemm_m_half
        tok = prompt_rows * w.S
        eta = tok / (tok + m_half) if m_half > 0 else 1.0
        pt_prefill = 1 if hw.tp_prefill_replicated > 0 else pt
        flops = tok * (2 * Lpp / pt_prefill) * sh.layer_flops_per_token(w.S) + prompt_rows * 2 * sh.V * sh.d / pt_prefill
        t_total = flops / (hw.flops_per_gpu * hw.sustained_flops_fraction * max(eta, 1e-6))
        cap = self._gen_concurrency(node, rows, w.S + self._mean_len() / 2.0)

        def step_overhead(live_rows: float) -> float:
            """What one decode step costs beyond its bytes at the memory rate: a constant (launch of the step's graph,
            sampling, bookkeeping), the latency of every layer's chain of dependent kernels, the per-row work of the
            element-wise kernels, and under tensor parallelism the two all-reduce launches per layer (one exchange
            while rows x ranks <= 256, reduce-scatter + all-gather above)."""
            t = hw.decode_step_overhead_s + Lpp * (hw.decode_layer_chain_s + hw.decode_row_layer_s * live_rows)
            if pt > 1 and hw.tp_decode_allreduce_s > 0:
                small = hw.tp_decode_allreduce_small_s > 0 and live_rows * pt <= 256
                t += 2 * Lpp * (hw.tp_decode_allreduce_small_s if small else hw.tp_decode_allreduce_s)
            return t

        backlog = 0.0                                                   # row-steps that waited for a free slot
        live_frac = 1.0
        sub = 32
        for frac, a, b in self._length_bins():
            steps = max(0, b - a)
            for i in range(sub):
                t_mid = a + (i + 0.5) * steps / sub
                dt = steps / sub
                live = rows * (live_frac - frac * (i + 0.5) / sub)
                run = min(live, cap)
                if live > cap:
                    backlog += (live - cap) * dt
                elif backlog > 0 and dt > 0:
                    extra = min(cap - live, backlog / dt)
                    backlog -= extra * dt
                    run = live + extra
                ctx = w.S * share + t_mid
                step_bytes = w_bytes / e_w + run * kv_tok * ctx / e_kv + 2 * run * sh.d * Lpp * sh.sb
                t_total += dt * (step_bytes / bw + step_overhead(run))
            live_frac -= frac
        if backlog > 0:                                                 # the rows that waited run on after the others
            ctx = w.S * share + self._mean_len() / 2.0
            step_bytes = w_bytes / e_w + cap * kv_tok * ctx / e_kv
            t_total += backlog / cap * (step_bytes / bw + step_overhead(cap))
        return t_total

    def _gen_concurrency(self, node: ExecNode, b: float, past: float) -> float:
        """Rows of one replica that decode together: the microbatch, capped by the generator's slots and by how
        many contexts of the mean length ``past`` fit into the paged KV pool."""
        hw, sh = self.hw, self._shape(node.model)
        c = b
        if hw.gen_max_concurrency > 0:
            c = min(c, hw.gen_max_concurrency)
        if hw.gen_kv_budget_bytes > 0:
            pd, pp, pt = node.pi
            per_token = 2 * (sh.d / pt) * sh.sb * (sh.L / pp)
            c = min(c, hw.gen_kv_budget_bytes / (per_token * max(1.0, past)))
        return max(1.0, c)

    def _engine_terms(self, node: ExecNode) -> float:
        """Time the reference's model leaves out and the engine spends: attention FLOPs below the GEMM rate,
        elementwise kernels, per-step overhead of the decode loop. All zero with the default hardware fields."""
        hw, sh, w = self.hw, self._shape(node.model), self.workload
        pd, pp, pt = node.pi
        P = pd * pp * pt
        extra = 0.0
        if node.role is Role.GENERATION:
            if node.n_active is None and self._length_bins() is not None:
                return 0.0                                   # _generation_time_by_lengths already counts the steps
            if hw.decode_step_overhead_s > 0:
                if node.phase_steps is not None:
                    steps, past = node.phase_steps, w.S + node.phase_t_start + node.phase_steps / 2
                else:
                    steps, past = w.T - 1, w.S + w.T / 2
                b = self._b_local(node)
                extra += hw.decode_step_overhead_s * steps * b / self._gen_concurrency(node, b, past) * self._effective_mb(node)
            return extra
        seq = self._seq_len(node)
        n = node.n_seqs if node.n_seqs is not None else w.B * w.K
        mult = 1.0 if node.role is Role.INFERENCE else (3.0 + float(self.activation_checkpointing))
        if hw.attention_flops_eff < 1.0:
            att = mult * n * seq * 2 * sh.L * seq * sh.d
            extra += att / (P * hw.flops_per_gpu * hw.sustained_flops_fraction) * (1.0 / hw.attention_flops_eff - 1.0)
        if hw.elementwise_s_per_token_layer > 0:
            extra += mult * n * seq * sh.L / P * hw.elementwise_s_per_token_layer
        return extra

    def _gemm_efficiency(self, node: ExecNode, m_rows: float) -> float:
        hw = self.hw
        eta = m_rows / (m_rows + hw.gemm_m_half) if hw.gemm_m_half > 0 else 1.0
        pt = node.pi[2]
        if pt > 1 and hw.gemm_k_half > 0:
            sh = self._shape(node.model)
            k_min = min(sh.d // pt, sh.f // pt)
            eta *= k_min / (k_min + hw.gemm_k_half)
        return eta

    def _generation_flops(self, node: ExecNode) -> float:
        hw, sh, w = self.hw, self._shape(node.model), self.workload
        pd, pp, pt = node.pi
        P = pd * pp * pt
        S, T = w.S, w.T
        Lpp = sh.L / pp
        b = self._b_local(node)
        if node.phase_steps is not None:
            steps, past, has_prefill = node.phase_steps, S + node.phase_t_start + node.phase_steps / 2, node.is_prefill_phase
        else:
            steps, past, has_prefill = T - 1, S + T / 2, True
        w_bytes = Lpp / pt * sh.layer_params * sh.sb
        ridge = hw.flops_per_gpu / hw.memory_bandwidth
        m_half = hw.gemm_m_half
        total_work = self._work(node)
        t_total, w_prefill = 0.0, 0.0
        if has_prefill:
            eta = b * S / (b * S + m_half) if m_half > 0 else 1.0
            flops = b * S * (2 * Lpp / pt) * sh.layer_flops_per_token(S)
            nbytes = w_bytes + 2 * b * S * sh.d * Lpp * sh.sb
            inten = flops / nbytes if nbytes > 0 else float("inf")
            F = hw.flops_per_gpu * hw.sustained_flops_fraction * eta if inten >= ridge else inten * hw.memory_bandwidth
            w_prefill = self._effective_batch(node) * (S * 2 * sh.L * sh.layer_flops_per_token(S) + 2 * sh.V * sh.d)
            t_total += w_prefill / (P * F) if F > 0 else 0.0
        if steps > 0:
            b = self._gen_concurrency(node, b, past)
            eta = b / (b + m_half) if m_half > 0 else 1.0
            flops = b * (2 * Lpp / pt) * sh.layer_flops_per_token(past)
            a_bytes = 2 * b * sh.d * Lpp * sh.sb
            kv_bytes = 2 * past * (sh.d / pt) * sh.sb * b * Lpp
            all_bytes = w_bytes + a_bytes + kv_bytes
            e_w = hw.decode_bw_eff
            e_kv = min(1.0, 3.5 * hw.decode_bw_eff)
            eff = (w_bytes * e_w + kv_bytes * e_kv + a_bytes) / all_bytes if all_bytes > 0 else e_w
            inten = flops / all_bytes if all_bytes > 0 else float("inf")
            F = hw.flops_per_gpu * eta if inten >= ridge else inten * hw.memory_bandwidth * eff
            t_total += (total_work - w_prefill) / (P * F) if F > 0 else 0.0
        return total_work / (P * t_total) if t_total > 0 else hw.flops_per_gpu

    # ------------------------------------------------------------------ non-GEMM overhead
    def _non_gemm(self, node: ExecNode) -> float:
        hw = self.hw
        if hw.non_gemm_constant == 0.0 and hw.non_gemm_scaling == 0.0:
            return 0.0
        if node.role is Role.GENERATION:
            return 0.0
        pd, pp, pt = node.pi
        Lpp = self._shape(node.model).L / pp
        scale = self._b_local(node) / hw.non_gemm_batch_cal if hw.non_gemm_batch_cal > 0 else 1.0
        at_tp = Lpp * (hw.non_gemm_constant + hw.non_gemm_scaling / pt)
        ideal = Lpp * (hw.non_gemm_constant + hw.non_gemm_scaling) / pt
        extra = (at_tp - ideal) * scale
        if node.role is Role.TRAINING:
            extra *= 3 + float(self.activation_checkpointing)
        return max(0.0, extra)

    # ------------------------------------------------------------------ communication
    def _collective(self, coll: Collective, M: float, allocs: Tuple[Allocation, ...], p: int) -> float:
        hw = self.hw
        if coll is Collective.P2P:
            a, b = hw.tier_p2p(allocs)
            return a + M * b
        a, b = hw.tier_coll(allocs)
        if hw.fabric == "nvswitch" and hw.tier_name(allocs) == "g":
            if p <= 1:
                return 0.0
            # one hop through the switch; all-reduce reduces in the switch (NVLS)
            if coll is Collective.ALLREDUCE:
                return a + M * b
            return a + (p - 1) / p * M * b
        if coll in (Collective.ALLGATHER, Collective.REDUCESCATTER):
            return (p - 1) * a + (p - 1) / p * M * b
        if coll is Collective.ALLREDUCE:
            return 2 * (p - 1) * a + 2 * (p - 1) / p * M * b
        return (p - 1) * a + M * b  # all-to-all

    def _intra_comm(self, node: ExecNode) -> float:
        hw, sh, w = self.hw, self._shape(node.model), self.workload
        role, model = node.role, node.model
        pd, pp, pt = node.pi
        m = self._effective_mb(node)
        BK, S, T = w.B * w.K, w.S, w.T
        alloc = node.allocs[0]
        hide = 1.0 - min(max(hw.fused_overlap, 0.0), 1.0)

        def tp_allreduce(M: float) -> float:
            if hw.fabric == "nvswitch":
                if pt > 1 and role is Role.GENERATION and hw.tp_decode_allreduce_s > 0 and M <= 8e6:
                    # one launch of the fused decode all-reduce: its time is flag exchanges and switch round trips,
                    # not bytes; nothing hides it, the next GEMM needs its result
                    return hw.tp_decode_allreduce_s + M * hw.beta_coll_g
                return 0.0 if pt <= 1 else hide * (hw.alpha_coll_g + M * hw.beta_coll_g)
            return 2 * (pt - 1) * hw.alpha_coll_g + 2 * (pt - 1) / pt * M * hw.beta_coll_g

        r_ext, n_ext, g_ext = alloc.extent
        s = g_ext // pt
        nodes_per_rep = math.ceil(pp / s) if s > 0 else pp
        edges = pp - 1
        inter = nodes_per_rep - 1
        intra = edges - inter
        tier = "r" if r_ext > 1 else ("n" if n_ext > 1 else "g")
        a_inter, b_inter = getattr(hw, f"alpha_p2p_{tier}"), getattr(hw, f"beta_p2p_{tier}")

        def pp_p2p(M: float, steps: float) -> float:
            if edges == 0 or steps == 0:
                return 0.0
            return (intra / edges * steps * (hw.alpha_p2p_g + M * hw.beta_p2p_g)
                    + inter / edges * steps * (a_inter + M * b_inter))

        Lpp = sh.L / pp
        act = lambda rows, tokens: rows * tokens * sh.d * sh.sb / (pd * m)  # noqa: E731
        if role is Role.GENERATION:
            if node.n_active is not None:
                n, steps = node.n_active, node.phase_steps
                cost = 0.0
                if node.is_prefill_phase:
                    cost += pp_p2p(act(n, S), m + pp - 2) + 2 * Lpp * m * tp_allreduce(act(n, S))
                return cost + pp_p2p(act(n, 1), steps * (m + pp - 2)) + 2 * steps * Lpp * m * tp_allreduce(act(n, 1))
            # with length quantiles and a measured launch time, the decode steps' all-reduces are counted step by step
            # (few rows: one exchange; many: two phases) in _generation_time_by_lengths
            by_steps = pt > 1 and hw.tp_decode_allreduce_s > 0 and hw.expected_lengths > 0 and self._length_bins() is not None
            decode_ar = 0.0 if by_steps else 2 * (T - 1) * Lpp * m * tp_allreduce(act(BK, 1))
            return (pp_p2p(act(BK, S), m + pp - 2) + pp_p2p(act(BK, 1), (T - 1) * (m + pp - 2))
                    + 2 * Lpp * m * tp_allreduce(act(BK, S)) + decode_ar)
        if role is Role.INFERENCE:
            n = node.n_seqs if node.n_seqs is not None else BK
            return pp_p2p(act(n, S + T), m + pp - 2) + 2 * Lpp * m * tp_allreduce(act(n, S + T))
        if role is Role.TRAINING:
            params = sh.params + (sh.d if model in (Model.CRITIC, Model.AC_SHARE) else 0)
            msg = params * sh.sb / (pp * pt)
            allocs = node.allocs
            if self.optimizer_stage == 0:
                dp = self._collective(Collective.ALLREDUCE, msg, allocs, pd)
            elif self.optimizer_stage == 1:
                dp = self._collective(Collective.ALLREDUCE, msg, allocs, pd) + self._collective(Collective.ALLGATHER, msg, allocs, pd)
            else:
                dp = self._collective(Collective.REDUCESCATTER, msg, allocs, pd) + self._collective(Collective.ALLGATHER, msg, allocs, pd)
            if hw.fabric == "nvswitch":
                dp *= hide
            n_coll = 4 + 2 * float(self.activation_checkpointing)
            return dp + pp_p2p(act(BK, S + T), m + 2 * pp - 3) + n_coll * Lpp * m * tp_allreduce(act(BK, S + T))
        raise ValueError(f"no communication model for role={role} model={model}")

    def _comm_time(self, node: ExecNode) -> float:
        a, b = self.hw.tier(node.allocs)
        modeled = a + node.payload_in_bytes / min(node.allocs[0].size(), node.allocs[1].size()) * b
        if str(node.label or "").startswith("W_"):
            return modeled * self.hw.weight_comm_scale
        return modeled + self.hw.activation_comm_overhead_s

    def _reshard_time(self, node: ExecNode) -> float:
        P = node.allocs[0].size()
        return self.hw.reshard_scale * self._collective(Collective.ALLTOALL, node.payload_in_bytes / P, node.allocs, P)
