"""User-facing training loops: ``GRPOTrainer``, ``PPOTrainer``, ``DPOTrainer``.

Each ``step`` takes its inputs as (pinned) host tensors, copies them to the GPU, runs one full
iteration of the algorithm on this rank's share of the batch and returns python floats read back
from the device, i.e. it is the end-to-end call a user makes. With a ``DPContext`` the ranks split
the prompts evenly, normalise losses by global counts and run the fused data-parallel optimizer.

Pipeline per iteration (vertex names of the RPEG templates in brackets):
  GRPO: generate [g_pi] -> reference log-probs [i_ref] -> rewards [i_R] -> group advantages ->
        policy step [t_pi] -> optimizer -> new weight version visible to the next generation.
  PPO : generate [g_pi] -> reference log-probs [i_ref], reward scores [i_R], values [i_V] -> GAE ->
        actor step [t_pi], critic step [t_V] -> optimizers.
  DPO : policy/reference sequence log-probs [i_pi, i_ref] -> pair loss -> policy step [t_pi].
Reference entry points: run_graph_grpo / run_graph_ppo / run_graph_dpo
(RPEG/runtime/algorithms/grpo_graph.py:25, ppo_graph.py:1072, dpo_graph.py:414).
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..models.llama import LlamaConfig, LlamaModel
from ..ops import kernels as K
from . import algorithms as A
from .generation import Generator
from .optimizer import AdamW


def _h2d(t: Optional[torch.Tensor], device, dtype=None) -> Optional[torch.Tensor]:
    if t is None:
        return None
    out = t.to(device, non_blocking=True)
    return out if dtype is None else out.to(dtype)


def balanced_groups(resp_lens: List[int], prompt_len: int, group: int, ranks: int) -> List[List[int]]:
    """Deal prompt groups (``group`` consecutive rows each) to ``ranks`` so that the token totals are as even as a
    greedy pass makes them: groups in order of decreasing tokens, each to the rank with the fewest tokens so far (ties
    to the lower rank, so every rank computes the same answer). Returns the sorted group indices of each rank."""
    n_groups = len(resp_lens) // group
    weight = [sum(prompt_len + int(l) for l in resp_lens[g * group:(g + 1) * group]) for g in range(n_groups)]
    load = [0] * ranks
    out: List[List[int]] = [[] for _ in range(ranks)]
    for g in sorted(range(n_groups), key=lambda g: (-weight[g], g)):
        r = min(range(ranks), key=lambda r: (load[r], r))
        out[r].append(g)
        load[r] += weight[g]
    return [sorted(gs) for gs in out]


class _Base:
    def __init__(self, device, dp=None):
        self.device = torch.device(device)
        self.dp = dp
        self.iteration = 0
        self.weight_version = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self._marks: List = []

    def _mark(self, name: str) -> None:
        """Record a CUDA event that closes phase ``name``; the phase times are read after the step's sync."""
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._marks.append((name, ev))

    def _phase_ms(self) -> Dict[str, float]:
        out: Dict[str, float] = {}
        for (_, a), (name, b) in zip(self._marks, self._marks[1:]):
            out[f"{name}_ms"] = out.get(f"{name}_ms", 0.0) + a.elapsed_time(b)
        if len(self._marks) > 1:
            # first mark (inputs are on the device) to last mark (the optimizer's last kernel)
            out["device_ms"] = self._marks[0][1].elapsed_time(self._marks[-1][1])
        self._marks = []
        return out

    @property
    def world(self) -> int:
        return 1 if self.dp is None else self.dp.world

    def _global_sum(self, value: float) -> float:
        if self.dp is None or self.dp.world == 1:
            return float(value)
        return self.dp.all_reduce_scalar(float(value))

    def _read(self, metrics: Dict[str, torch.Tensor]) -> Dict[str, float]:
        keys = list(metrics)
        packed = torch.stack([metrics[k].reshape(()).float() for k in keys]).cpu()
        self.d2h_bytes = packed.numel() * 4
        return {k: float(v) for k, v in zip(keys, packed.tolist())}


class GRPOTrainer(_Base):
    def __init__(self, cfg: LlamaConfig, *, device="cuda:0", samples_per_prompt: int = 8, max_new: int = 2048,
                 prompt_len: int = 512, algo: Optional[A.AlgoConfig] = None, lr: float = 1e-6, gen_slots: int = 64,
                 kv_budget_bytes: float = 40e9, recompute: str = "full", dp=None, seed: int = 0, eos_id: int = 2,
                 sync_interval: int = 8, use_graphs: bool = True, gen_tp: bool = False, tp_comm: Optional[str] = None,
                 group_attention: bool = False, gen_tp_size: Optional[int] = None):
        """``gen_tp``: generate tensor parallel over all ranks of ``dp`` (every rank decodes ALL rows of the global batch
        on 1/world of the weights and KV heads, ``models.tp_decode``) while the reference pass, the policy update and the
        optimizer stay data parallel; ``gen_slots`` is then the number of rows of the whole batch decoded at once.
        ``gen_tp_size`` (a divisor of the world size, default: all ranks): generation layout ``(world / t, 1, t)``, i.e.
        groups of ``t`` consecutive ranks decode the rows of their own prompts tensor parallel; ``gen_slots`` then counts
        the rows of one group."""
        super().__init__(device, dp)
        self.cfg = cfg
        self.K = samples_per_prompt
        self.max_new = max_new
        self.algo = algo or A.AlgoConfig(kl_coef=0.04)
        self.seed = seed
        self.gen_tp = bool(gen_tp) and dp is not None and dp.world > 1
        self.overlap_grad_reduce = True
        tp = dp.world if self.gen_tp else 1
        self.tp_group, self.tp_rank, self.tp_index = (dp.group if dp is not None else None), (dp.rank if dp is not None else 0), 0
        if self.gen_tp and gen_tp_size is not None and int(gen_tp_size) != dp.world:
            import torch.distributed as dist
            tp = int(gen_tp_size)
            if tp < 2 or dp.world % tp:
                raise ValueError(f"gen_tp_size={gen_tp_size} must be a divisor (>= 2) of the {dp.world} ranks")
            base = dist.get_process_group_ranks(dp.group) if dp.group is not None else list(range(dp.world))
            for gi in range(dp.world // tp):               # every rank creates every group, in the same order
                grp = dist.new_group([base[gi * tp + j] for j in range(tp)])
                if gi == dp.rank // tp:
                    self.tp_group = grp
            self.tp_rank, self.tp_index = dp.rank % tp, dp.rank // tp
        self.tp = tp
        # Gradients are dead while generating and the KV cache is dead while training, so both live
        # in one arena sized for the larger of the two.
        from ..models.llama import ParamLayout
        n_par = ParamLayout(cfg).total
        kv_need = min(int(kv_budget_bytes), Generator.kv_bytes_for(cfg, gen_slots, prompt_len + max_new, tp))
        arena_bytes = max(4 * n_par, kv_need)
        multi = dp is not None and dp.world > 1
        w = dp.alloc_weights(cfg) if multi else None
        if multi:
            g = dp.alloc_grads(cfg, extra_bytes=arena_bytes)
            arena = dp.buffers[f"{dp.tag}.g"].bytes_view
        else:
            arena = torch.zeros(arena_bytes, dtype=torch.uint8, device=self.device)
            g = arena[: 4 * n_par].view(torch.float32)
        self.actor = LlamaModel(cfg, self.device, trainable=True, recompute=recompute, weights=w, grads=g, seed=seed)
        if w is not None:
            self.actor.init_weights(seed)
        self.ref = LlamaModel(cfg, self.device, weights=None, seed=seed)
        self.ref.load_flat(self.actor)
        self.opt = AdamW(self.actor, lr=lr, dp=dp)
        self.gen_model = self.actor
        if self.gen_tp:
            from ..models.tp_decode import TPDecodeModel
            self.gen_model = TPDecodeModel(self.actor, self.tp_group, max_batch=gen_slots, comm_mode=tp_comm)
            layout = f"tp{tp}" if tp == dp.world else f"dp{dp.world // tp} x tp{tp}"
            self.parallelism = f"generation {layout} ({self.gen_model.comm.backend}), reference + training dp{dp.world}"
        self.gen = Generator(self.gen_model, max_slots=gen_slots, max_seq_len=prompt_len + max_new, eos_id=eos_id,
                             sync_interval=sync_interval, use_graphs=use_graphs,
                             kv_storage=arena[: arena_bytes // 2 * 2].view(torch.bfloat16),
                             group_attention=group_attention and samples_per_prompt > 1)
        self.last_counters: Dict[str, float] = {}
        self.last_reshard_us: Optional[float] = None

    def _all_ranks(self, t: torch.Tensor) -> torch.Tensor:
        """Rows of every rank of this rank's tensor-parallel generation group, in rank order (the group generates the
        rows of all its members; with one group that is the whole batch)."""
        import torch.distributed as dist
        t = t.contiguous()
        out = torch.empty((self.tp * t.shape[0], *t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t, group=self.tp_group)
        return out

    def step(self, prompts: torch.Tensor, rewards: Optional[torch.Tensor] = None,
             forced_lens: Optional[torch.Tensor] = None) -> Dict[str, float]:
        """``prompts [B_local, S]`` int32 host tensor; ``rewards [B_local*K]`` host tensor standing in
        for the reward model (one scalar per sample) ; ``forced_lens [B_local*K]`` optional EOS positions."""
        t0 = time.perf_counter()
        self.h2d_bytes = prompts.numel() * prompts.element_size()
        p_dev = _h2d(prompts, self.device, torch.int32)
        B, S = p_dev.shape
        N = B * self.K
        rep = p_dev.repeat_interleave(self.K, dim=0).contiguous()
        self._mark("begin")
        if self.gen_tp:
            from .generation import GenerationResult
            f_all = None
            if forced_lens is not None:
                f_all = self._all_ranks(torch.as_tensor(forced_lens, dtype=torch.int32).to(self.device)).tolist()
            rep_all = self._all_ranks(rep)
            whole = self.gen.generate(rep_all, self.max_new, temperature=self.algo.temperature,
                                      seed=self.seed + 100003 * self.iteration + 7919 * self.tp_index, forced_lens=f_all,
                                      group_size=self.K)
            # Every rank holds every row now, so the rows of the data-parallel phases (reference pass, policy update)
            # are dealt out by TOKENS rather than by position: whole prompt groups, heaviest first, each to the rank
            # with the least work so far. The phases end when their slowest rank does.
            mine = balanced_groups(whole.lengths.tolist(), S, self.K, self.tp)[self.tp_rank]
            rows = torch.tensor([g * self.K + j for g in mine for j in range(self.K)], dtype=torch.long, device=self.device)
            gen = GenerationResult(whole.tokens[rows].contiguous(), whole.logprobs[rows].contiguous(),
                                   whole.lengths[rows].contiguous(), whole.counters)
            rep = rep_all[rows].contiguous()
            if rewards is not None:
                self.h2d_bytes += rewards.numel() * rewards.element_size()
                rewards = self._all_ranks(_h2d(rewards, self.device, torch.float32))[rows].contiguous()
            N = int(rows.numel())
        else:
            gen = self.gen.generate(rep, self.max_new, temperature=self.algo.temperature,
                                    seed=self.seed + 100003 * self.iteration, forced_lens=forced_lens, group_size=self.K)
        resp_lens = gen.lengths.tolist()
        self._mark("generate")
        ro = A.Rollout(rep, [S] * N, gen.tokens, resp_lens, gen.logprobs, gen.response_mask(),
                       weight_version=self.weight_version)
        if self.algo.kl_coef != 0.0:
            ro.ref_logp = A.sequence_logprobs(self.ref, ro, self.algo)
        self._mark("reference")
        if rewards is None:
            raise ValueError("GRPOTrainer.step needs per-sample rewards (the reward model's output)")
        if not self.gen_tp:
            self.h2d_bytes += rewards.numel() * rewards.element_size()
        ro.scores = _h2d(rewards, self.device, torch.float32)
        A.grpo_advantages(ro, self.K)
        denom = self._global_sum(ro.n_response_tokens())
        self.actor.zero_grad()
        # data parallel: finished layers' gradients are reduced in buckets under the rest of the last backward pass
        hook = self.dp.overlap_hook(self.opt, self.actor) if (self.world > 1 and self.overlap_grad_reduce) else None
        m = A.policy_train_step(self.actor, ro, self.algo, denom_tokens=denom, on_last_backward=hook)
        self._mark("train")
        # data parallel: the time up to the first barrier of the step is the wait for the slowest rank's backward
        self.opt.step(after_wait=(lambda: self._mark("grad_wait")) if self.world > 1 else None)
        self._mark("optimizer")
        if self.gen_tp:
            self.gen_model.refresh()      # layout switch: the updated replicated weights -> this rank's generation shards
            self._mark("reshard")
        self.weight_version += 1
        self.iteration += 1
        m["grad_norm"] = self.opt.grad_norm()
        out = self._read(m)
        out.update(self._phase_ms())
        if self.gen_tp:
            self.last_reshard_us = self.gen_model.last_reshard_us
            out["reshard_us"] = float(self.last_reshard_us or 0.0)
        out.update(samples=float(N), gen_tokens=float(sum(resp_lens)), train_tokens=float(sum(ro.total_lens())),
                   wall_s=time.perf_counter() - t0)
        self.last_counters = dict(gen.counters)
        return out


class DPOTrainer(_Base):
    def __init__(self, cfg: LlamaConfig, *, device="cuda:0", algo: Optional[A.AlgoConfig] = None, lr: float = 1e-6,
                 recompute: str = "full", dp=None, seed: int = 0):
        super().__init__(device, dp)
        self.cfg = cfg
        self.algo = algo or A.AlgoConfig(beta=0.1)
        w = dp.alloc_weights(cfg) if (dp is not None and dp.world > 1) else None
        g = dp.alloc_grads(cfg) if (dp is not None and dp.world > 1) else None
        self.policy = LlamaModel(cfg, self.device, trainable=True, recompute=recompute, weights=w, grads=g, seed=seed)
        if w is not None:
            self.policy.init_weights(seed)
        self.ref = LlamaModel(cfg, self.device, seed=seed)
        self.ref.load_flat(self.policy)
        self.opt = AdamW(self.policy, lr=lr, dp=dp)

    def step(self, prompt_ids: torch.Tensor, resp_ids: torch.Tensor, resp_lens: Optional[torch.Tensor] = None) -> Dict[str, float]:
        """``prompt_ids [2P, S]`` (each prompt twice), ``resp_ids [2P, T]`` interleaved chosen/rejected."""
        t0 = time.perf_counter()
        self.h2d_bytes = prompt_ids.numel() * prompt_ids.element_size() + resp_ids.numel() * resp_ids.element_size()
        p_dev = _h2d(prompt_ids, self.device, torch.int32)
        r_dev = _h2d(resp_ids, self.device, torch.int32)
        N, S = p_dev.shape
        T = r_dev.shape[1]
        self._mark("begin")
        lens = [T] * N if resp_lens is None else [int(x) for x in resp_lens.tolist()]
        lens_t = torch.tensor(lens, device=self.device)
        mask = (torch.arange(T, device=self.device)[None, :] < lens_t[:, None]).float()
        ro = A.Rollout(p_dev, [S] * N, r_dev, lens, torch.zeros((N, T), dtype=torch.float32, device=self.device), mask)
        ref_lp = A.sequence_logprobs(self.ref, ro, self.algo)
        ref_seq = K.masked_rowsum(ref_lp, mask)
        self._mark("reference")
        pairs = int(self._global_sum(N // 2))
        self.policy.zero_grad()
        m = A.dpo_train_step(self.policy, ro, ref_seq, self.algo, n_pairs_global=pairs)
        self._mark("train")
        self.opt.step()
        self._mark("optimizer")
        self.iteration += 1
        self.weight_version += 1
        m["grad_norm"] = self.opt.grad_norm()
        out = self._read(m)
        out.update(self._phase_ms())
        out.update(samples=float(N // 2), train_tokens=float(sum(ro.total_lens())), wall_s=time.perf_counter() - t0)
        return out


class PPOTrainer(_Base):
    """Actor + reference + critic + reward model. ``share_actor_critic=True`` trains one trunk with
    an LM head and a value head (the AC-share template) instead of a separate critic."""

    def __init__(self, cfg: LlamaConfig, *, device="cuda:0", max_new: int = 512, prompt_len: int = 128,
                 algo: Optional[A.AlgoConfig] = None, lr_actor: float = 1e-6, lr_critic: float = 5e-6,
                 gen_slots: int = 64, kv_budget_bytes: float = 20e9, recompute: str = "full", dp=None, seed: int = 0,
                 eos_id: int = 2, share_actor_critic: bool = False, reward_cfg: Optional[LlamaConfig] = None,
                 sync_interval: int = 8, use_graphs: bool = True):
        super().__init__(device, dp)
        from dataclasses import replace
        self.cfg = cfg
        self.max_new = max_new
        self.algo = algo or A.AlgoConfig()
        self.seed = seed
        self.shared = share_actor_critic
        actor_cfg = replace(cfg, lm_head=True, scalar_head=share_actor_critic)
        head_cfg = replace(cfg, lm_head=False, scalar_head=True)
        multi = dp is not None and dp.world > 1
        self.actor = LlamaModel(actor_cfg, self.device, trainable=True, recompute=recompute,
                                weights=dp.alloc_weights(actor_cfg) if multi else None,
                                grads=dp.alloc_grads(actor_cfg) if multi else None, seed=seed)
        if multi:
            self.actor.init_weights(seed)
        self.ref = LlamaModel(replace(cfg, lm_head=True, scalar_head=False), self.device, seed=seed)
        self.ref.w[: self.ref.layout.total].copy_(self.actor.w[: self.ref.layout.total])
        self.critic = None
        if not share_actor_critic:
            self.critic = LlamaModel(head_cfg, self.device, trainable=True, recompute=recompute,
                                     weights=dp.alloc_weights(head_cfg, tag="critic") if multi else None,
                                     grads=dp.alloc_grads(head_cfg, tag="critic") if multi else None, seed=seed + 1)
            if multi:
                self.critic.init_weights(seed + 1)
        r_cfg = replace(reward_cfg or cfg, lm_head=False, scalar_head=True)
        self.reward = LlamaModel(r_cfg, self.device, seed=seed + 2)
        self.opt_actor = AdamW(self.actor, lr=lr_actor, dp=dp)
        self.opt_critic = AdamW(self.critic, lr=lr_critic, dp=dp.clone("critic") if multi else None) if self.critic else None
        self.gen = Generator(self.actor, max_slots=gen_slots, max_seq_len=prompt_len + max_new,
                             kv_budget_bytes=kv_budget_bytes, eos_id=eos_id, sync_interval=sync_interval,
                             use_graphs=use_graphs)
        self.last_counters: Dict[str, float] = {}

    def step(self, prompts: torch.Tensor, forced_lens: Optional[torch.Tensor] = None) -> Dict[str, float]:
        t0 = time.perf_counter()
        self.h2d_bytes = prompts.numel() * prompts.element_size()
        p_dev = _h2d(prompts, self.device, torch.int32).contiguous()
        N, S = p_dev.shape
        self._mark("begin")
        gen = self.gen.generate(p_dev, self.max_new, temperature=self.algo.temperature,
                                seed=self.seed + 100003 * self.iteration, forced_lens=forced_lens)
        resp_lens = gen.lengths.tolist()
        self._mark("generate")
        ro = A.Rollout(p_dev, [S] * N, gen.tokens, resp_lens, gen.logprobs, gen.response_mask(),
                       weight_version=self.weight_version)
        ro.ref_logp = A.sequence_logprobs(self.ref, ro, self.algo)
        self._mark("reference")
        ro.scores = A.reward_scores(self.reward, ro, self.algo)
        self._mark("reward")
        ro.values = A.critic_values(self.actor if self.shared else self.critic, ro, self.algo)
        A.ppo_targets(ro, self.algo)
        self._mark("values")
        denom = self._global_sum(ro.n_response_tokens())
        self.actor.zero_grad()
        m = A.policy_train_step(self.actor, ro, self.algo, denom_tokens=denom, value_model_shared=self.shared)
        self._mark("train")
        self.opt_actor.step()
        self._mark("optimizer")
        if self.critic is not None:
            self.critic.zero_grad()
            m.update(A.critic_train_step(self.critic, ro, self.algo, denom_tokens=denom))
            self._mark("critic_train")
            self.opt_critic.step()
            self._mark("critic_optimizer")
        self.weight_version += 1
        self.iteration += 1
        m["grad_norm"] = self.opt_actor.grad_norm()
        m["mean_score"] = ro.scores.mean()
        out = self._read(m)
        out.update(self._phase_ms())
        out.update(samples=float(N), gen_tokens=float(sum(resp_lens)), train_tokens=float(sum(ro.total_lens())),
                   wall_s=time.perf_counter() - t0)
        self.last_counters = dict(gen.counters)
        return out


class PipelineGRPOTrainer(_Base):
    """GRPO whose policy update is PIPELINE parallel over all ranks while generation and the reference pass stay data
    parallel: the plan ``g_pi, i_ref: (dp, pp, tp) = (G, 1, 1)``, ``t_pi: (1, G, 1)``.

    Every rank keeps the whole bf16 policy (``actor``, what the generator and nothing else reads) and a frozen
    reference copy, but gradients, fp32 master weights and Adam moments only for ITS pipeline stage: the stage model's
    weights are a view into the whole policy's flat buffer (a stage's parameters are one contiguous range of it), so
    the optimizer writes the updated stage where the generator will read it. One iteration:

        generate this rank's prompts (K samples each) -> reference log-probs of its rows        data parallel
        all-gather the rollouts: every stage needs every microbatch                            NCCL all-gather, a few MB
        group advantages, 1F1B policy step over the global batch (``parallel.pp``)             pipeline parallel
        Adam on the stage, clipped by the norm of the WHOLE model                              one all-reduce of a scalar
        layout switch: every stage's range is broadcast into all ranks' whole policy           NCCL broadcast per stage

    Compared with the data-parallel trainer a rank holds 1/G of the gradients and optimizer state without any
    gradient reduction; the price is the pipeline bubble and the weight broadcast (the reference's in-place layout
    switch between a training and a generation layout, RPEG/runtime/semantic_worker.py:5503-5872, with Megatron's
    1F1B schedule for the update, RPEG/runtime/workers/megatron_worker.py:1657,3808)."""

    def __init__(self, cfg: LlamaConfig, *, device="cuda:0", samples_per_prompt: int = 8, max_new: int = 2048,
                 prompt_len: int = 512, algo: Optional[A.AlgoConfig] = None, lr: float = 1e-6, gen_slots: int = 64,
                 kv_budget_bytes: float = 40e9, recompute: str = "full", seed: int = 0, eos_id: int = 2,
                 sync_interval: int = 8, use_graphs: bool = True, group=None):
        import torch.distributed as dist

        from ..models.llama import ParamLayout
        from ..parallel.pp import PipelineRunner
        super().__init__(device, None)
        if not dist.is_initialized():
            raise RuntimeError("PipelineGRPOTrainer needs an initialised process group (one rank per stage)")
        self.group = group
        self.rank, self.n_stages = dist.get_rank(group), dist.get_world_size(group)
        if cfg.tie_embeddings:
            raise ValueError("tied embeddings put one matrix on two stages; not supported by the pipeline trainer")
        if cfg.n_layers < self.n_stages:
            raise ValueError(f"{cfg.n_layers} layers cannot fill {self.n_stages} pipeline stages")
        self.cfg, self.K, self.max_new, self.seed = cfg, samples_per_prompt, max_new, seed
        self.algo = algo or A.AlgoConfig(kl_coef=0.04)
        full = ParamLayout(cfg)
        # (offset, length) of every stage inside the whole model's flat buffer
        self.spans: List[tuple] = []
        for s in range(self.n_stages):
            lay = ParamLayout(cfg, (s, self.n_stages))
            base = full.entries[next(iter(lay.entries))][0]
            for name, (off, shape) in lay.entries.items():
                if full.entries[name] != (base + off, shape):
                    raise AssertionError(f"stage {s}: {name} is not where the whole model keeps it")
            self.spans.append((base, lay.total))
        base, n_stage = self.spans[self.rank]
        self.full_w = torch.empty(full.total, dtype=torch.bfloat16, device=self.device)
        self.actor = LlamaModel(cfg, self.device, weights=self.full_w, seed=seed)
        self.actor.init_weights(seed)                                  # same seed, same weights on every rank
        self.ref = LlamaModel(cfg, self.device, seed=seed)
        self.ref.load_flat(self.actor)
        self.stage = LlamaModel(cfg, self.device, trainable=True, recompute=recompute, stage=(self.rank, self.n_stages),
                                weights=self.full_w[base:base + n_stage], seed=seed)
        self.opt = AdamW(self.stage, lr=lr, norm_group=group if group is not None else dist.group.WORLD)
        self.opt.shard_off = base                                      # where this stage's optimizer state sits in the whole flat space
        self.runner = PipelineRunner(self.stage, group)
        self.gen = Generator(self.actor, max_slots=gen_slots, max_seq_len=prompt_len + max_new, kv_budget_bytes=kv_budget_bytes,
                             eos_id=eos_id, sync_interval=sync_interval, use_graphs=use_graphs)
        self._scalar = torch.zeros(1, dtype=torch.float64, device=self.device)
        self.published_bytes = 0
        self.last_counters: Dict[str, float] = {}

    @property
    def world(self) -> int:
        return self.n_stages

    def _global_sum(self, value: float) -> float:
        import torch.distributed as dist
        self._scalar.fill_(float(value))
        dist.all_reduce(self._scalar, group=self.group)
        return float(self._scalar.item())

    def _gather(self, t: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist
        t = t.contiguous()
        out = torch.empty((self.n_stages * t.shape[0], *t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t, group=self.group)
        return out

    def gather_rollout(self, ro: A.Rollout) -> A.Rollout:
        """The rollouts of all ranks, in rank order (every rank holds the same number of rows)."""
        lens = self._gather(torch.tensor(ro.resp_lens, dtype=torch.int32, device=self.device)).tolist()
        plens = self._gather(torch.tensor(ro.prompt_lens, dtype=torch.int32, device=self.device)).tolist()
        g = lambda t: None if t is None else self._gather(t)
        return A.Rollout(g(ro.prompt_ids), plens, g(ro.resp_ids), lens, g(ro.old_logp), g(ro.mask), g(ro.ref_logp), g(ro.values),
                         g(ro.scores), None, None, ro.weight_version)

    def train_policy(self, ro_global: A.Rollout, denom_tokens: float) -> Dict[str, torch.Tensor]:
        """One optimizer step on a GLOBAL rollout (the same on every stage): 1F1B forward/backward, Adam on the stage."""
        self.stage.zero_grad()
        m = A.policy_train_step(self.stage, ro_global, self.algo, denom_tokens=denom_tokens, pipeline=self.runner)
        self.opt.step()
        return m

    def publish(self) -> int:
        """Layout switch after an update: every stage's range of the whole policy goes to all ranks. Returns the bytes
        this rank received."""
        import torch.distributed as dist
        got = 0
        for s, (base, n) in enumerate(self.spans):
            src = dist.get_global_rank(self.group, s) if self.group is not None else s
            dist.broadcast(self.full_w[base:base + n], src=src, group=self.group)
            if s != self.rank:
                got += 2 * n
        self.published_bytes += got
        return got

    def step(self, prompts: torch.Tensor, rewards: Optional[torch.Tensor] = None,
             forced_lens: Optional[torch.Tensor] = None) -> Dict[str, float]:
        """``prompts [B_local, S]`` and ``rewards [B_local * K]``: THIS rank's share, as for the data-parallel trainer."""
        t0 = time.perf_counter()
        self.h2d_bytes = prompts.numel() * prompts.element_size()
        p_dev = _h2d(prompts, self.device, torch.int32)
        B, S = p_dev.shape
        N = B * self.K
        rep = p_dev.repeat_interleave(self.K, dim=0).contiguous()
        self._mark("begin")
        gen = self.gen.generate(rep, self.max_new, temperature=self.algo.temperature, seed=self.seed + 100003 * self.iteration + self.rank,
                                forced_lens=forced_lens, group_size=self.K)
        resp_lens = gen.lengths.tolist()
        self._mark("generate")
        ro = A.Rollout(rep, [S] * N, gen.tokens, resp_lens, gen.logprobs, gen.response_mask(), weight_version=self.weight_version)
        if self.algo.kl_coef != 0.0:
            ro.ref_logp = A.sequence_logprobs(self.ref, ro, self.algo)
        self._mark("reference")
        if rewards is None:
            raise ValueError("PipelineGRPOTrainer.step needs per-sample rewards (the reward model's output)")
        self.h2d_bytes += rewards.numel() * rewards.element_size()
        ro.scores = _h2d(rewards, self.device, torch.float32)
        glob = self.gather_rollout(ro)
        A.grpo_advantages(glob, self.K)
        m = self.train_policy(glob, float(glob.n_response_tokens()))
        self._mark("train")
        self.publish()
        self._mark("publish")
        self.weight_version += 1
        self.iteration += 1
        m["grad_norm"] = self.opt.grad_norm()
        out = self._read(m)
        out.update(self._phase_ms())
        out.update(samples=float(N), gen_tokens=float(sum(resp_lens)), train_tokens=float(sum(ro.total_lens())),
                   wall_s=time.perf_counter() - t0)
        self.last_counters = dict(gen.counters)
        return out
