"""Alpha-beta hardware description used by the cost and memory models.

The field set and tier selection follow the reference (RPEG/model/hardware.py:18-122): peak FLOP/s,
HBM capacity and bandwidth, alpha/beta for collectives and point-to-point on three tiers (inside a
node ``g``, across nodes ``n``, across racks ``r``), GEMM saturation constants, decode bandwidth
efficiency, non-GEMM per-layer costs and the run-time correction scales.

Two additions describe an NVSwitch machine such as an 8xB200 node:
  * ``fabric="nvswitch"`` replaces the ring collective formulas inside a node with switch ones
    (every GPU reaches every peer at full link bandwidth; all-reduce can reduce in the switch);
  * ``fused_overlap`` in [0, 1] is the measured fraction of a tensor-parallel or data-parallel
    collective that the fused compute+collective kernels hide behind math.
A third group ("engine terms") prices what this framework's engine does differently from the reference's
assumptions: a three-matrix MLP, sustained instead of burst GEMM rate, attention and elementwise kernels at their
own measured rates, and a generator whose concurrency is bounded by its slots and its paged KV pool.
"""
from __future__ import annotations

from dataclasses import dataclass, fields, replace
from typing import Iterable, Tuple

from ..core.types import Allocation


@dataclass(frozen=True)
class Hardware:
    flops_per_gpu: float
    memory_per_gpu: float
    memory_bandwidth: float
    alpha_coll_g: float
    beta_coll_g: float
    alpha_coll_n: float
    beta_coll_n: float
    alpha_coll_r: float
    beta_coll_r: float
    alpha_p2p_g: float
    beta_p2p_g: float
    alpha_p2p_n: float
    beta_p2p_n: float
    alpha_p2p_r: float
    beta_p2p_r: float
    gemm_m_half: float = 5.0
    gemm_k_half: float = 0.0
    decode_bw_eff: float = 0.15
    non_gemm_constant: float = 0.0
    non_gemm_scaling: float = 0.0
    non_gemm_batch_cal: float = 64
    op_generation_scale: float = 1.0
    op_inference_scale: float = 1.0
    op_training_scale: float = 1.0
    activation_comm_overhead_s: float = 0.0
    weight_comm_scale: float = 1.0
    reshard_scale: float = 1.0
    # --- NVSwitch / fused-kernel extensions (defaults keep the reference's ring model exactly)
    fabric: str = "ring"
    fused_overlap: float = 0.0
    # --- engine terms, measured by calibrate.py on this framework's kernels (defaults reproduce the reference's
    #     model exactly; see NodeCostModel._engine_terms)
    ffn_matrices: float = 2.0                  # 3 for the gated (SwiGLU) MLP the engine runs
    sustained_flops_fraction: float = 1.0      # long compute-bound operators run under the power cap
    attention_flops_eff: float = 1.0           # fraction of the GEMM rate that attention FLOPs reach
    elementwise_s_per_token_layer: float = 0.0 # norms, RoPE, SwiGLU, residual adds: seconds per token and layer (forward)
    gen_max_concurrency: float = 0.0           # generator slots: rows decoding at once per replica (0 = whole batch)
    gen_kv_budget_bytes: float = 0.0           # paged KV pool per GPU; caps the concurrency by the mean context (0 = no cap)
    decode_step_overhead_s: float = 0.0        # per decode step: graph launch, sampling, bookkeeping
    tp_decode_allreduce_s: float = 0.0         # > 0: measured time of ONE fused all-reduce + residual + RMSNorm launch of the
    #                                            tensor-parallel decode step (latency bound: two flag exchanges and a switch
    #                                            round trip); replaces the alpha-beta estimate for decode-sized messages
    tp_decode_allreduce_small_s: float = 0.0   # > 0: the same for rows x ranks <= 256, where the launch is ONE exchange
    #                                            (self-validating units pushed to every rank, reduced locally)
    tp_prefill_replicated: float = 0.0         # > 0: a tensor-parallel generation group prefills its prompts on every member
    #                                            (the engine's generator does; the reference's model shards the prefill)
    decode_layer_chain_s: float = 0.0          # per decode step and layer: latency of the chain of dependent kernels of a
    #                                            layer (what a step costs beyond its bytes at the copy rate, at any batch)
    decode_row_layer_s: float = 0.0            # per decode step, layer and live row: the per-row work of the element-wise
    #                                            kernels and of the GEMMs' second activation tile
    dp_reduce_gbs: float = 0.0                 # > 0: measured rate (GB/s of gradient bytes entering a rank) of the fused
    #                                            data-parallel gradient reduction; reported by calibrate.py
    expected_lengths: float = 0.0              # > 0: unsplit vertices are priced with the workload's length quantiles
    #                                            (rows stop at their own length) instead of every row running to the cap
    gen_shared_prompt_cost: float = 1.0        # < 1: the K samples of a prompt share its KV pages; a shared prompt token
    #                                            costs this fraction of a private one per decode step, prefill runs once per prompt

    @staticmethod
    def _span(allocs: Iterable[Allocation]) -> Tuple[int, int]:
        allocs = tuple(allocs)
        racks = max(a.origin[0] + a.extent[0] for a in allocs) - min(a.origin[0] for a in allocs)
        nodes = max(a.origin[1] + a.extent[1] for a in allocs) - min(a.origin[1] for a in allocs)
        return racks, nodes

    def tier_name(self, allocs: Iterable[Allocation]) -> str:
        racks, nodes = self._span(allocs)
        return "r" if racks > 1 else ("n" if nodes > 1 else "g")

    def tier_coll(self, allocs: Iterable[Allocation]) -> Tuple[float, float]:
        t = self.tier_name(allocs)
        return getattr(self, f"alpha_coll_{t}"), getattr(self, f"beta_coll_{t}")

    def tier_p2p(self, allocs: Iterable[Allocation]) -> Tuple[float, float]:
        t = self.tier_name(allocs)
        return getattr(self, f"alpha_p2p_{t}"), getattr(self, f"beta_p2p_{t}")

    def tier(self, allocs: Iterable[Allocation]) -> Tuple[float, float]:
        return self.tier_p2p(allocs)

    def with_updates(self, **kw) -> "Hardware":
        return replace(self, **kw)

    @classmethod
    def field_names(cls) -> Tuple[str, ...]:
        return tuple(f.name for f in fields(cls))


def b200_nvswitch(flops: float = 1.37e15, hbm_bw: float = 6.5e12, mem: float = 180e9,
                  link_bw: float = 770e9, allreduce_busbw: float = 725e9) -> Hardware:
    """One 8xB200 NVSwitch node: measured sustained bf16 GEMM rate, STREAM-style HBM copy rate,
    peer copy 770 GB/s per direction, 8-rank all-reduce bus bandwidth 725 GB/s. The inter-node and
    inter-rack tiers are filled with a 400 Gb/s-per-GPU network so multi-node plans stay priceable."""
    ib = 1.0 / 50e9
    return Hardware(
        flops_per_gpu=flops, memory_per_gpu=mem, memory_bandwidth=hbm_bw,
        alpha_coll_g=6e-6, beta_coll_g=1.0 / allreduce_busbw,
        alpha_coll_n=25e-6, beta_coll_n=ib, alpha_coll_r=40e-6, beta_coll_r=2 * ib,
        alpha_p2p_g=4e-6, beta_p2p_g=1.0 / link_bw,
        alpha_p2p_n=15e-6, beta_p2p_n=ib, alpha_p2p_r=30e-6, beta_p2p_r=2 * ib,
        gemm_m_half=96.0, gemm_k_half=0.0, decode_bw_eff=0.6,
        fabric="nvswitch", fused_overlap=0.0,
    )
