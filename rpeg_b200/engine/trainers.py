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
                 sync_interval: int = 8, use_graphs: bool = True):
        super().__init__(device, dp)
        self.cfg = cfg
        self.K = samples_per_prompt
        self.max_new = max_new
        self.algo = algo or A.AlgoConfig(kl_coef=0.04)
        self.seed = seed
        # Gradients are dead while generating and the KV cache is dead while training, so both live
        # in one arena sized for the larger of the two.
        from ..models.llama import ParamLayout
        n_par = ParamLayout(cfg).total
        kv_need = min(int(kv_budget_bytes), Generator.kv_bytes_for(cfg, gen_slots, prompt_len + max_new))
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
        self.gen = Generator(self.actor, max_slots=gen_slots, max_seq_len=prompt_len + max_new, eos_id=eos_id,
                             sync_interval=sync_interval, use_graphs=use_graphs,
                             kv_storage=arena[: arena_bytes // 2 * 2].view(torch.bfloat16))
        self.last_counters: Dict[str, float] = {}

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
        self.h2d_bytes += rewards.numel() * rewards.element_size()
        ro.scores = _h2d(rewards, self.device, torch.float32)
        A.grpo_advantages(ro, self.K)
        denom = self._global_sum(ro.n_response_tokens())
        self.actor.zero_grad()
        m = A.policy_train_step(self.actor, ro, self.algo, denom_tokens=denom)
        self._mark("train")
        self.opt.step()
        self._mark("optimizer")
        self.weight_version += 1
        self.iteration += 1
        m["grad_norm"] = self.opt.grad_norm()
        out = self._read(m)
        out.update(self._phase_ms())
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
        lens = [T] * N if resp_lens is None else [int(x) for x in resp_lens.tolist()]
        lens_t = torch.tensor(lens, device=self.device)
        mask = (torch.arange(T, device=self.device)[None, :] < lens_t[:, None]).float()
        ro = A.Rollout(p_dev, [S] * N, r_dev, lens, torch.zeros((N, T), dtype=torch.float32, device=self.device), mask)
        ref_lp = A.sequence_logprobs(self.ref, ro, self.algo)
        ref_seq = K.masked_rowsum(ref_lp, mask)
        pairs = int(self._global_sum(N // 2))
        self.policy.zero_grad()
        m = A.dpo_train_step(self.policy, ro, ref_seq, self.algo, n_pairs_global=pairs)
        self.opt.step()
        self.iteration += 1
        self.weight_version += 1
        m["grad_norm"] = self.opt.grad_norm()
        out = self._read(m)
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
        gen = self.gen.generate(p_dev, self.max_new, temperature=self.algo.temperature,
                                seed=self.seed + 100003 * self.iteration, forced_lens=forced_lens)
        resp_lens = gen.lengths.tolist()
        ro = A.Rollout(p_dev, [S] * N, gen.tokens, resp_lens, gen.logprobs, gen.response_mask(),
                       weight_version=self.weight_version)
        ro.ref_logp = A.sequence_logprobs(self.ref, ro, self.algo)
        ro.scores = A.reward_scores(self.reward, ro, self.algo)
        ro.values = A.critic_values(self.actor if self.shared else self.critic, ro, self.algo)
        A.ppo_targets(ro, self.algo)
        denom = self._global_sum(ro.n_response_tokens())
        self.actor.zero_grad()
        m = A.policy_train_step(self.actor, ro, self.algo, denom_tokens=denom, value_model_shared=self.shared)
        self.opt_actor.step()
        if self.critic is not None:
            self.critic.zero_grad()
            m.update(A.critic_train_step(self.critic, ro, self.algo, denom_tokens=denom))
            self.opt_critic.step()
        self.weight_version += 1
        self.iteration += 1
        m["grad_norm"] = self.opt_actor.grad_norm()
        m["mean_score"] = ro.scores.mean()
        out = self._read(m)
        out.update(samples=float(N), gen_tokens=float(sum(resp_lens)), train_tokens=float(sum(ro.total_lens())),
                   wall_s=time.perf_counter() - t0)
        self.last_counters = dict(gen.counters)
        return out
