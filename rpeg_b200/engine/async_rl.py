"""Disaggregated GRPO with bounded staleness: generation ranks and training ranks are disjoint sets of GPUs that
run concurrently and meet only through versioned peer-memory channels (``parallel.publish``).

Iteration ``k`` (1-based):

    generation ranks   wait for weight version max(0, k - 1 - tau)  -> generate their share of the B * K rows with it
                       -> scatter the rows (ids, sampling log-probs, lengths) to the trainer that owns each global
                          row index -> raise the rollout version to k
    training ranks     wait for rollout version k -> reference log-probs -> group advantages -> clipped policy step
                       (data parallel among the trainers, fused reduce-scatter + Adam + all-gather) -> push the new
                       weights (every trainer a share) into every generation rank's slot k % (tau + 2) -> raise the
                       weight version to k

With ``tau = 0`` the two sides alternate (on-policy); with ``tau >= 1`` generation of iteration ``k + 1`` overlaps
training of iteration ``k`` and the policy loss corrects for the lag through the importance ratio against the
log-probs recorded at sampling time. A generation rank keeps ``tau + 2`` weight slots; its models are views of
the slots, so pushed weights are used where they land and are never copied again. The first GEMM of a generation
phase carries the version gate of its slot.

Reference: bounded staleness in RPEG/passes/unroll.py:62-152 (publisher selection) and
RPEG/runtime/weight_versions.py:25 (consumer version), shadow weight copies on disjoint allocations in
RPEG/search/evaluate.py:115-141, asynchronous weight transfer in RPEG/runtime/semantic_worker.py:6289-6535.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..models.llama import LlamaConfig, LlamaModel, ParamLayout
from ..ops import kernels as K
from ..parallel.publish import RolloutChannel, WeightChannel, consumed_version
from . import algorithms as A
from .generation import Generator
from .optimizer import AdamW


class AsyncGRPO:
    def __init__(self, cfg: LlamaConfig, *, gen_ranks: Sequence[int], train_ranks: Sequence[int], prompts_per_step: int,
                 samples_per_prompt: int = 8, max_new: int = 256, prompt_len: int = 64, tau: int = 1,
                 algo: Optional[A.AlgoConfig] = None, lr: float = 1e-6, gen_slots: int = 64, kv_budget_bytes: float = 16e9,
                 seed: int = 0, eos_id: int = 2, device="cuda:0", wait_timeout_s: float = 600.0, use_graphs: bool = True):
        if set(gen_ranks) & set(train_ranks):
            raise ValueError("staleness needs disjoint generation and training ranks")
        self.cfg, self.tau = cfg, tau
        self.device = torch.device(device)
        self.rank = dist.get_rank()
        self.gen_ranks, self.train_ranks = list(gen_ranks), list(train_ranks)
        self.is_gen, self.is_train = self.rank in self.gen_ranks, self.rank in self.train_ranks
        self.K, self.max_new, self.prompt_len = samples_per_prompt, max_new, prompt_len
        self.algo = algo or A.AlgoConfig(kl_coef=0.04)
        self.seed, self.timeout = seed, wait_timeout_s
        self.n_rows = prompts_per_step * samples_per_prompt
        if self.n_rows % len(self.gen_ranks) or self.n_rows % len(self.train_ranks):
            raise ValueError("B * K must divide by the number of generation ranks and of training ranks")
        n_par = ParamLayout(cfg).total
        self.weights = WeightChannel(n_par, self.device, None, self.train_ranks, self.gen_ranks, tau)
        self.rollouts = RolloutChannel(self.n_rows, max_new, self.device, None, self.gen_ranks, self.train_ranks, tau)
        train_group = dist.new_group(self.train_ranks)            # collective over all ranks
        self.step_no = 0
        self.counters: Dict[str, float] = {}
        self.last_lengths: List[int] = []
        self.waited_for_rollouts_s = 0.0
        if self.is_gen:
            kv = torch.zeros(int(min(kv_budget_bytes, Generator.kv_bytes_for(cfg, gen_slots, prompt_len + max_new))) // 2,
                             dtype=torch.bfloat16, device=self.device)
            self.models: List[LlamaModel] = []
            self.generators: List[Generator] = []
            for s in range(self.weights.slots):
                m = LlamaModel(cfg, self.device, weights=self.weights.slot_weights(s), seed=seed)
                self.models.append(m)
                self.generators.append(Generator(m, max_slots=gen_slots, max_seq_len=prompt_len + max_new, eos_id=eos_id,
                                                 use_graphs=use_graphs, kv_storage=kv))
            self.models[0].init_weights(seed)                      # version 0 = the common initial weights
        if self.is_train:
            from ..parallel.dp import DPContext
            multi = len(self.train_ranks) > 1
            self.dp = DPContext(self.device, train_group) if multi else None
            w = self.dp.alloc_weights(cfg) if multi else None
            g = self.dp.alloc_grads(cfg) if multi else None
            self.actor = LlamaModel(cfg, self.device, trainable=True, weights=w, grads=g, seed=seed)
            self.actor.init_weights(seed)
            self.ref = LlamaModel(cfg, self.device, seed=seed)
            self.ref.load_flat(self.actor)
            self.opt = AdamW(self.actor, lr=lr, dp=self.dp)
        torch.cuda.synchronize(self.device)
        dist.barrier()

    # ------------------------------------------------------------------ one iteration on this rank's side
    def step(self, prompts: torch.Tensor, rewards: torch.Tensor, forced_lens=None) -> Dict[str, float]:
        """``prompts [B, S]`` int32 and ``rewards [B * K]`` fp32 are the GLOBAL host tensors of this iteration (the
        same on every rank; each rank takes the rows it owns). ``forced_lens [B * K]`` optionally fixes the EOS
        position of every row (synthetic length control). Returns this rank's metrics."""
        self.step_no += 1
        k = self.step_no
        t0 = time.perf_counter()
        out = self._generate(k, prompts, forced_lens) if self.is_gen else self._train(k, prompts, rewards)
        out["wall_s"] = time.perf_counter() - t0
        out["step"] = float(k)
        return out

    def _rows_of(self, index: int, parts: int) -> range:
        per = self.n_rows // parts
        return range(index * per, (index + 1) * per)

    def _generate(self, k: int, prompts: torch.Tensor, forced_lens=None) -> Dict[str, float]:
        v = consumed_version(k, self.tau)
        t0 = time.perf_counter()
        if v > 0 and not self.weights.ready(v, self.timeout):
            raise TimeoutError(f"weight version {v} did not arrive within {self.timeout} s")
        waited = time.perf_counter() - t0
        slot = v % self.weights.slots
        model, gen = self.models[slot], self.generators[slot]
        if v > 0:
            model.weight_gate = self.weights.gate(v)
        rows = self._rows_of(self.gen_ranks.index(self.rank), len(self.gen_ranks))
        rep = prompts.to(self.device, torch.int32).repeat_interleave(self.K, dim=0)[rows.start:rows.stop].contiguous()
        forced = None if forced_lens is None else [int(x) for x in forced_lens[rows.start:rows.stop]]
        res = gen.generate(rep, self.max_new, temperature=self.algo.temperature, seed=self.seed + 100003 * k + self.rank,
                           forced_lens=forced, group_size=self.K if (rows.start % self.K == 0 and len(rows) % self.K == 0) else 1)
        idx = torch.arange(rows.start, rows.stop, dtype=torch.int64, device=self.device)
        self.rollouts.send(k, idx, res.tokens, res.logprobs, res.lengths)
        K.check_status()
        self.counters = dict(res.counters)
        self.last_lengths = [int(x) for x in res.lengths.tolist()]
        return {"role": 0.0, "weight_version": float(v), "gen_tokens": float(res.lengths.sum().item()),
                "waited_for_weights_s": waited}

    def collect(self, k: int, prompts: torch.Tensor) -> A.Rollout:
        """Training side, first half of iteration ``k``: wait for the rollouts of ``k``, take this rank's rows and
        compute their reference log-probs. ``self.waited_for_rollouts_s`` holds the time spent waiting."""
        t0 = time.perf_counter()
        if not self.rollouts.ready(k, self.timeout):
            raise TimeoutError(f"rollouts of iteration {k} did not arrive within {self.timeout} s")
        self.waited_for_rollouts_s = time.perf_counter() - t0
        ids, logp, lens = self.rollouts.receive(k)
        rows = self._rows_of(self.train_ranks.index(self.rank), len(self.train_ranks))
        rep = prompts.to(self.device, torch.int32).repeat_interleave(self.K, dim=0)[rows.start:rows.stop].contiguous()
        resp_lens = [int(x) for x in lens.tolist()]
        T = self.max_new
        mask = (torch.arange(T, device=self.device)[None, :] < lens[:, None]).float()
        ro = A.Rollout(rep, [rep.shape[1]] * rep.shape[0], ids.clone(), resp_lens, logp.clone(), mask,
                       weight_version=consumed_version(k, self.tau))
        if self.algo.kl_coef != 0.0:
            ro.ref_logp = A.sequence_logprobs(self.ref, ro, self.algo)
        return ro

    def update(self, k: int, ro: A.Rollout) -> Dict[str, float]:
        """Training side, second half: group advantages from ``ro.scores``, the clipped policy step (data parallel among
        the trainers), and the push of weight version ``k`` to every generation rank."""
        A.grpo_advantages(ro, self.K)
        denom = float(ro.n_response_tokens())
        if self.dp is not None:
            denom = self.dp.all_reduce_scalar(denom)
        self.actor.zero_grad()
        m = A.policy_train_step(self.actor, ro, self.algo, denom_tokens=denom)
        self.opt.step()
        self.weights.publish(self.actor.w, k)
        K.check_status()
        return {"role": 1.0, "samples": float(ro.n), "loss": float(m["loss"]), "grad_norm": float(self.opt.grad_norm()), "trained_on_version": float(ro.weight_version),
                "published_version": float(k), "train_tokens": float(sum(ro.total_lens())), "waited_for_rollouts_s": self.waited_for_rollouts_s}

    def _train(self, k: int, prompts: torch.Tensor, rewards: torch.Tensor) -> Dict[str, float]:
        ro = self.collect(k, prompts)
        rows = self._rows_of(self.train_ranks.index(self.rank), len(self.train_ranks))
        ro.scores = rewards[rows.start:rows.stop].to(self.device, torch.float32)
        return self.update(k, ro)

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        dist.barrier()
        self.weights.close()
        self.rollouts.close()
