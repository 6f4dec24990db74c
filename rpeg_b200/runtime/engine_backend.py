"""Engine backend: gives the nodes of a runtime graph their meaning on the GPU.

Every rank (one process per GPU) executes the same graph in the same order; an operator node runs the
engine call of its vertex on this rank's share of the batch:

  g_pi / g_ac   paged-KV generation with CUDA-graph decode              (engine.generation.Generator)
  i_ref         frozen reference log-probs                               (algorithms.sequence_logprobs)
  i_R           reward model scores, or a rule-based reward without one  (algorithms.reward_scores)
  i_V / i_ac    critic / shared-trunk values                             (algorithms.critic_values)
  i_pi          policy sequence log-probs of preference pairs (DPO)
  t_pi / t_ac   policy (or shared trunk) update incl. optimizer step     (algorithms.policy_train_step / dpo_train_step)
  t_V           critic update incl. optimizer step                       (algorithms.critic_train_step)

The plan must be synchronous (tau = 0) and of one of two families on all GPUs of the node. Data parallel
(every vertex pp = tp = 1): weights are replicated in symmetric memory and updated in place by the fused
optimizer, so COMM and RESHARD nodes between vertices move nothing and only report their payload. Pipeline-trained
(GRPO; generation and inference data parallel, training vertices pp = G): the update runs 1F1B over all ranks
(``engine.trainers.PipelineGRPOTrainer``), each rank keeps gradients and optimizer state of its stage only, and the
layout switch back to the replicated generation copy (a broadcast per stage) runs at the end of the training node.
Generation is continuously batched, so the quantile phases of a split generation vertex are not
separate decode loops: the first phase node generates every row, and each phase node *emits* the rows
whose length falls into its interval (what downstream split inference nodes consume).
Checkpoints use the flat-shard format (``runtime.checkpoint``): bf16 weights from rank 0, the fp32
master/m/v shards from every rank with their global offsets, so a resumed job may use another
data-parallel degree. Reference entry points: run_graph_ppo / run_graph_grpo / run_graph_dpo
(RPEG/runtime/algorithms/ppo_graph.py:1072, grpo_graph.py:25, dpo_graph.py:414).
"""
from __future__ import annotations

import asyncio
import json
import os
from pathlib import Path
from typing import Any, Dict, List, Optional

from ..passes.lower import ExecNodeType
from . import checkpoint as ckpt
from .containers import ContainerRef, WeightVersion
from .errors import RuntimeConfigError, RuntimeExecutionError
from .executor import NodeExecutionResult, model_name, node_step, split_part_index
from .weight_versions import consumer_weight_version as consumed_version_of


def llama_config_from_run(m, max_pos: int, **kw):
    from ..models.llama import LlamaConfig
    heads = m.num_heads or (m.hidden_dim // m.head_dim)
    return LlamaConfig(n_layers=m.layers, d_model=m.hidden_dim, d_ff=m.ffn_dim, n_heads=heads,
                       n_kv_heads=m.num_kv_heads or heads, head_dim=m.head_dim, vocab=m.vocab_size, rms_eps=m.rms_eps,
                       rope_theta=m.rope_theta, max_pos=max_pos, **kw)


def disaggregated_ranks(compiled):
    """``(generation ranks, training ranks)`` when the plan puts every generation vertex, data parallel, on one set of GPUs
    of the node and every other vertex, data parallel, on the remaining GPUs; ``None`` for any other plan."""
    from ..core.types import Role
    cfg = compiled.config
    if compiled.device_space.R * compiled.device_space.N != 1:
        return None
    sets = {"gen": set(), "rest": set()}
    for v in cfg.rpeg.vertices:
        devs = {c[2] for c in cfg.plan.sigma[v.id].coords()}
        dp, pp, tp = cfg.plan.pi[v.id]
        if pp != 1 or tp != 1 or dp != len(devs):
            return None
        key = "gen" if v.kind.role is Role.GENERATION else "rest"
        if sets[key] and sets[key] != devs:
            return None
        sets[key] = devs
    gen, rest = sets["gen"], sets["rest"]
    if not gen or not rest or gen & rest or len(gen | rest) != compiled.device_space.G:
        return None
    return sorted(gen), sorted(rest)


def validate_engine_plan(compiled) -> str:
    """The plan families this backend executes, both on all ``G`` GPUs of the node. Returns the family:

      ``"data_parallel"``    every vertex ``(dp, pp, tp) = (G, 1, 1)``
      ``"pipeline_train"``   generation / inference vertices ``(G, 1, 1)``, every training vertex ``(1, G, 1)`` (GRPO):
                             the update runs 1F1B over all ranks as stages, the publication edge is a real layout
                             switch (stage weights broadcast into the replicated generation copy)
      ``"tp_generation"``    the generation vertex ``(G / t, 1, t)``, t >= 2: groups of t consecutive GPUs decode the rows of
                             their prompts on 1/t of the weights and KV heads each (``models.tp_decode``; t = G: every GPU
                             decodes the whole batch), every other vertex ``(G, 1, 1)`` (GRPO); the RESHARD node of
                             the publication edge re-slices the updated weights into the generation layout
      ``"disaggregated"``    generation data parallel on some GPUs, everything else data parallel on the others (GRPO),
                             any staleness ``tau >= 0``: the two sides run concurrently and meet through versioned
                             peer-memory channels (``engine.async_rl.AsyncGRPO``)"""
    from ..core.types import Role
    cfg = compiled.config
    g = compiled.device_space.num_devices()
    split = disaggregated_ranks(compiled)
    if split is not None:
        if compiled.run_config.algorithm.name != "grpo":
            raise RuntimeConfigError("engine backend: generation and training on disjoint GPUs is implemented for GRPO only")
        if compiled.run_config.checkpoints.resume_from:
            raise RuntimeConfigError("engine backend: a run with generation and training on disjoint GPUs cannot resume from a checkpoint")
        # This family writes no tensor checkpoints, so a replay would "restore" nothing: the engine would keep its
        # advanced weights, Adam state and version words and apply the replayed updates a second time.
        if int(compiled.run_config.monitoring.graph_replay_retries) > 0:
            raise RuntimeConfigError("engine backend: monitoring.graph_replay_retries > 0 is not supported with generation and "
                                     "training on disjoint GPUs (no checkpoint to replay from); set it to 0")
        return "disaggregated"
    train = [v for v in cfg.rpeg.vertices if v.kind.role is Role.TRAINING]
    piped = g > 1 and bool(train) and all(tuple(cfg.plan.pi[v.id]) == (1, g, 1) for v in train)
    gens = [v for v in cfg.rpeg.vertices if v.kind.role is Role.GENERATION]
    gen_pis = {tuple(cfg.plan.pi[v.id]) for v in gens}
    tp_gen = (g > 1 and len(gen_pis) == 1 and next(iter(gen_pis))[1] == 1 and next(iter(gen_pis))[2] >= 2
              and next(iter(gen_pis))[0] * next(iter(gen_pis))[2] == g)
    for v in cfg.rpeg.vertices:
        dp, pp, tp = cfg.plan.pi[v.id]
        if (piped and v in train) or (tp_gen and v in gens):
            continue
        if pp != 1 or tp != 1 or dp != g:
            raise RuntimeConfigError(f"engine backend runs data-parallel plans, or data-parallel generation with pipeline-parallel "
                                     f"training: {v.id} has (dp,pp,tp)=({dp},{pp},{tp}) on {g} GPU(s); expected ({g},1,1)"
                                     + (f" or, for training vertices, (1,{g},1)" if g > 1 else ""))
    if piped:
        if compiled.run_config.algorithm.name != "grpo":
            raise RuntimeConfigError("engine backend: pipeline-parallel training vertices are implemented for GRPO only")
        layers = compiled.run_config.models["actor"].layers
        if layers < g:
            raise RuntimeConfigError(f"engine backend: {layers} layers cannot fill {g} pipeline stages")
    if any(int(t) > 0 for t in cfg.rpeg.tau.values()):
        raise RuntimeConfigError("engine backend: staleness (tau > 0) needs generation and training on disjoint GPUs "
                                 "(optimizer.plan_family: disaggregated)")
    if float(getattr(compiled.run_config.algorithm, "entropy_coef", 0.0) or 0.0) != 0.0 and compiled.run_config.algorithm.name == "dpo":
        raise RuntimeConfigError("engine backend: algorithm.entropy_coef applies to the PPO / GRPO policy objective, not to DPO; set it to 0")
    if tp_gen:
        if piped:
            raise RuntimeConfigError("engine backend: tensor-parallel generation with pipeline-parallel training is not a supported combination")
        if compiled.run_config.algorithm.name != "grpo":
            raise RuntimeConfigError("engine backend: a tensor-parallel generation vertex is implemented for GRPO only")
        return "tp_generation"
    return "pipeline_train" if piped else "data_parallel"


class EngineOperationHandler:
    def __init__(self, compiled, attempt: int = 0):
        import torch
        import torch.distributed as dist
        from ..engine import algorithms as A
        self.family = validate_engine_plan(compiled)
        self.compiled, self.attempt = compiled, attempt
        self.torch, self.A = torch, A
        run = compiled.run_config
        self.run = run
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        if self.world != compiled.device_space.num_devices():
            raise RuntimeConfigError(f"run file plans {compiled.device_space.num_devices()} GPU(s) but WORLD_SIZE={self.world}")
        self.device = torch.device(f"cuda:{int(os.environ.get('LOCAL_RANK', '0'))}")
        torch.cuda.set_device(self.device)
        self.dp = None
        if self.world > 1:
            if not dist.is_initialized():
                dist.init_process_group("nccl", device_id=self.device)
            if self.family in ("data_parallel", "tp_generation"):
                from ..parallel.dp import DPContext
                self.dp = DPContext(self.device)
        a, w, rt, o = run.algorithm, run.workload, run.runtime, run.optimizer_runtime
        self.algo_name = a.name
        # width of a tensor-parallel generation group (the world size unless the plan says (G / t, 1, t))
        self.gen_tp_size = 1
        if self.family == "tp_generation":
            from ..core.types import Role
            self.gen_tp_size = int(next(tuple(compiled.config.plan.pi[v.id]) for v in compiled.config.rpeg.vertices
                                        if v.kind.role is Role.GENERATION)[2])
        self.shared = any(v.id == "g_ac" for v in compiled.config.rpeg.vertices)
        self.algo = A.AlgoConfig(clip_eps=a.clip, kl_coef=a.kl_coef, beta=a.beta, gamma=a.gamma, gae_lambda=a.gae_lambda,
                                 value_coef=a.value_coef, entropy_coef=a.entropy_coef, temperature=a.temperature,
                                 micro_tokens=rt.micro_tokens)
        max_pos = w.context_length + w.generation_length
        cfg = llama_config_from_run(run.models["actor"], max_pos)
        from ..engine.trainers import DPOTrainer, GRPOTrainer, PPOTrainer
        common = dict(device=self.device, algo=self.algo, dp=self.dp, recompute=rt.recompute, seed=a.seed)
        self.async_engine = None
        if self.family == "disaggregated":
            from ..core.types import Model
            from ..engine.async_rl import AsyncGRPO
            gen_ranks, train_ranks = disaggregated_ranks(compiled)
            self.tau = int(compiled.config.rpeg.tau.get(Model.ACTOR, 0))
            kv = float(getattr(run.hardware, "kv_cache_budget_bytes", 0) or 16e9)
            self.async_engine = AsyncGRPO(cfg, gen_ranks=gen_ranks, train_ranks=train_ranks, prompts_per_step=w.batch_size,
                                          samples_per_prompt=w.samples_per_prompt, max_new=w.generation_length,
                                          prompt_len=w.context_length, tau=self.tau, algo=self.algo, lr=o.learning_rate_actor,
                                          gen_slots=rt.gen_slots, kv_budget_bytes=kv, seed=a.seed, eos_id=run.tokenizer.eos_token_id,
                                          device=self.device, use_graphs=rt.use_cuda_graphs, wait_timeout_s=float(rt.node_timeout_s or 600.0))
            self.trainer = None
        elif self.family == "pipeline_train":
            from ..engine.trainers import PipelineGRPOTrainer
            self.trainer = PipelineGRPOTrainer(cfg, device=self.device, algo=self.algo, recompute=rt.recompute, seed=a.seed,
                                               samples_per_prompt=w.samples_per_prompt, max_new=w.generation_length,
                                               prompt_len=w.context_length, lr=o.learning_rate_actor, gen_slots=rt.gen_slots,
                                               eos_id=run.tokenizer.eos_token_id, use_graphs=rt.use_cuda_graphs)
        elif a.name == "grpo":
            self.trainer = GRPOTrainer(cfg, samples_per_prompt=w.samples_per_prompt, max_new=w.generation_length,
                                       prompt_len=w.context_length, lr=o.learning_rate_actor, gen_slots=rt.gen_slots,
                                       eos_id=run.tokenizer.eos_token_id, use_graphs=rt.use_cuda_graphs,
                                       gen_tp=self.family == "tp_generation",
                                       gen_tp_size=(self.gen_tp_size if 1 < self.gen_tp_size < self.world else None), **common)
        elif a.name == "ppo":
            r = run.models.get("reward")
            self.trainer = PPOTrainer(cfg, max_new=w.generation_length, prompt_len=w.context_length, lr_actor=o.learning_rate_actor,
                                      lr_critic=o.learning_rate_critic, gen_slots=rt.gen_slots, eos_id=run.tokenizer.eos_token_id,
                                      share_actor_critic=self.shared, use_graphs=rt.use_cuda_graphs,
                                      reward_cfg=llama_config_from_run(r, max_pos) if r is not None else None, **common)
        else:
            self.trainer = DPOTrainer(cfg, lr=o.learning_rate_actor, **common)
        self.latest: Dict[str, int] = {}
        self.steps: Dict[int, Dict[str, Any]] = {}
        self.gen_cpu = torch.Generator().manual_seed(run.data.data_seed)
        self.vocab = cfg.vocab

    # ------------------------------------------------------------------ data
    def _local(self, n: int) -> slice:
        per = n // self.world
        return slice(self.rank * per, (self.rank + 1) * per)

    def _prompts(self, step: int):
        """Synthetic prompts of the workload's shape (every rank draws the global batch from the same
        seed and keeps its slice), or rows of token ids from ``data.train_prompts`` (JSONL)."""
        torch, w = self.torch, self.run.workload
        if self.run.data.train_prompts:
            rows = [json.loads(l) for l in open(self.run.resolve(self.run.data.train_prompts)) if l.strip()]
            ids = [r["input_ids"] if isinstance(r, dict) else r for r in rows]
            start = ((step - 1) * w.batch_size) % max(1, len(ids))
            batch = [ids[(start + i) % len(ids)] for i in range(w.batch_size)]
            t = torch.full((w.batch_size, w.context_length), self.run.tokenizer.pad_token_id, dtype=torch.int32)
            for i, r in enumerate(batch):
                r = r[-w.context_length:]
                t[i, w.context_length - len(r):] = torch.tensor(r, dtype=torch.int32)
        else:
            g = torch.Generator().manual_seed(self.run.data.data_seed * 1000003 + step)
            t = torch.randint(3, self.vocab, (w.batch_size, w.context_length), generator=g, dtype=torch.int32)
        return t[self._local(w.batch_size)].contiguous()

    def _state(self, step: int) -> Dict[str, Any]:
        return self.steps.setdefault(step, {})

    # ------------------------------------------------------------------ operators
    def _generate(self, st, step: int) -> Dict[str, Any]:
        tr, A, torch, w = self.trainer, self.A, self.torch, self.run.workload
        tp_gen = self.family == "tp_generation"
        sl = self._local(w.batch_size)
        K_ = w.samples_per_prompt
        rows_local = slice(sl.start * K_, sl.stop * K_)
        # a tensor-parallel generation group works on the prompts of ALL its members (t = world: the whole batch) on every
        # member; the data-parallel vertices after it take their slice of the result
        t = self.gen_tp_size if tp_gen else 1
        gi = self.rank // t if tp_gen else 0
        per_group = w.batch_size * t // self.world if tp_gen else w.batch_size
        group = slice(gi * per_group, (gi + 1) * per_group)                # prompts of this rank's group
        rows_group = slice(group.start * K_, group.stop * K_)
        if tp_gen and not self.run.data.train_prompts:
            prompts = self._prompts_global(step)[group].to(self.device)
        else:
            prompts = self._prompts(step).to(self.device)
            if tp_gen:
                prompts = tr._all_ranks(prompts)                            # gathered over the group
        rep = prompts.repeat_interleave(K_, dim=0).contiguous()
        a = self.run.algorithm
        forced = None
        if self.run.data.synthetic_response_lengths == "quantiles" and w.gen_quantiles:
            from .data import quantile_lengths
            rows = w.batch_size * K_                                        # drawn for the global batch, cut like the prompts
            all_lens = quantile_lengths(rows, w.quantile_tuples(), seed=self.run.data.data_seed * 1000003 + step)
            forced = all_lens[rows_group] if tp_gen else all_lens[rows_local]
        gen = tr.gen.generate(rep, w.generation_length, temperature=a.temperature, greedy=a.greedy,
                              seed=a.seed + 100003 * step + 7919 * gi, group_size=K_, top_k=a.top_k, top_p=a.top_p, forced_lens=forced)
        if tp_gen:
            from ..engine.generation import GenerationResult
            mine = slice(rows_local.start - rows_group.start, rows_local.stop - rows_group.start)
            gen = GenerationResult(gen.tokens[mine].contiguous(), gen.logprobs[mine].contiguous(),
                                   gen.lengths[mine].contiguous(), gen.counters)
            rep = rep[mine].contiguous()
        lens = gen.lengths.tolist()
        st["rollout"] = A.Rollout(rep, [w.context_length] * rep.shape[0], gen.tokens, lens, gen.logprobs, gen.response_mask(),
                                  weight_version=self.latest.get("ac_share" if self.shared else "actor", 0))
        st["lens"] = lens
        c = {k: v for k, v in gen.counters.items()}
        c.update(generated_tokens=int(sum(lens)), prompt_tokens=int(rep.numel()))
        return c

    def _emitted(self, st, node) -> int:
        """Rows of this rank whose generated length falls into the node's quantile phase."""
        part = split_part_index(node.node_id)
        lens = st.get("lens")
        if lens is None:
            return 0
        q = self.compiled.workload.gen_quantiles
        if part is None or not q:
            return len(lens)
        lo = q[part - 1][1] if part > 0 else 0
        hi = q[part][1]
        return sum(1 for l in lens if lo < l <= hi)

    def _prompts_global(self, step: int):
        """The whole synthetic prompt batch of a step (every rank draws the same one)."""
        torch, w = self.torch, self.run.workload
        g = torch.Generator().manual_seed(self.run.data.data_seed * 1000003 + step)
        return torch.randint(3, self.vocab, (w.batch_size, w.context_length), generator=g, dtype=torch.int32)

    def _run_op_disaggregated(self, node) -> Dict[str, Any]:
        """Generation ranks execute the generation vertices, training ranks everything else; a vertex of the other side
        is a no-op here (its effect reaches this rank through the versioned channels: a generation rank waits for the
        weight version its iteration consumes, a training rank for the rollouts of its iteration)."""
        eng, torch, w = self.async_engine, self.torch, self.run.workload
        step = node_step(node) or 1
        st = self._state(step)
        vid = node.vertex_id
        c: Dict[str, Any] = {"side": "generation" if eng.is_gen else "training"}
        if vid == "t_pi" and step == int(self.run.training.max_steps):
            self._leave_together = True                   # see execute(): no rank exits while a peer may still write to it
        if vid == "g_pi":
            if not eng.is_gen:
                return c
            if "generated" not in st:
                forced = None
                if self.run.data.synthetic_response_lengths == "quantiles" and w.gen_quantiles:
                    from .data import quantile_lengths
                    forced = quantile_lengths(w.batch_size * w.samples_per_prompt, w.quantile_tuples(), seed=self.run.data.data_seed * 1000003 + step)
                eng.step_no = step
                out = eng._generate(step, self._prompts_global(step), forced)
                st["generated"], st["lens"] = True, list(eng.last_lengths)
                c.update({k: v for k, v in eng.counters.items()})
                c.update(generated_tokens=int(out["gen_tokens"]), waited_for_weights_s=out["waited_for_weights_s"])
            c.update(emitted_rows=self._emitted(st, node), data_parallel_ranks=len(eng.gen_ranks),
                     weight_version=int(consumed_version_of(step, self.tau)), model="actor", shadow=self.tau > 0)
            return c
        if not eng.is_train:
            return c
        if vid not in ("i_ref", "i_R", "t_pi"):
            raise RuntimeExecutionError(f"engine backend (disaggregated GRPO) has no operator for vertex {vid}")
        # The inference vertices of a step may be dispatched in any order (and in quantile parts): whichever comes first
        # receives the step's rollouts (waiting for the generation ranks) and computes the reference log-probs.
        if "rollout" not in st:
            eng.step_no = step
            st["rollout"] = eng.collect(step, self._prompts_global(step))
            c["waited_for_rollouts_s"] = eng.waited_for_rollouts_s
        ro = st["rollout"]
        if ro.scores is None:                               # rule-based stand-in: shorter completions score higher
            ro.scores = -torch.tensor(ro.resp_lens, dtype=torch.float32, device=self.device) / w.generation_length
        if vid == "t_pi":
            out = eng.update(step, ro)
            c.update({k: out[k] for k in ("loss", "grad_norm", "trained_on_version", "published_version", "train_tokens")})
            c["optimizer_steps"] = 1
        return c

    def _run_op(self, node) -> Dict[str, Any]:
        if self.family == "disaggregated":
            return self._run_op_disaggregated(node)
        tr, A, torch = self.trainer, self.A, self.torch
        step = node_step(node) or 1
        st = self._state(step)
        vid, part = node.vertex_id, split_part_index(node.node_id)
        first = part in (None, 0)
        c: Dict[str, Any] = {}
        if vid in ("g_pi", "g_ac"):
            if "rollout" not in st:
                c.update(self._generate(st, step))
            c["emitted_rows"] = self._emitted(st, node)        # this rank's rows; the batch is cut evenly over the ranks
            c["data_parallel_ranks"] = self.world
        elif vid == "i_ref":
            if self.algo_name == "dpo":
                self._dpo_inputs(st, step)
                if "ref_seq" not in st:
                    from ..ops import kernels as K
                    st["ref_seq"] = K.masked_rowsum(A.sequence_logprobs(tr.ref, st["rollout"], self.algo), st["rollout"].mask)
            elif "ref" not in st:
                st["rollout"].ref_logp = A.sequence_logprobs(tr.ref, st["rollout"], self.algo)
                st["ref"] = True
        elif vid == "i_R":
            if "scores" not in st:
                ro = st["rollout"]
                if hasattr(tr, "reward"):
                    ro.scores = A.reward_scores(tr.reward, ro, self.algo)
                else:   # rule-based stand-in: shorter completions score higher, deterministic per row
                    ro.scores = -torch.tensor(st["lens"], dtype=torch.float32, device=self.device) / self.run.workload.generation_length
                st["scores"] = True
        elif vid in ("i_V", "i_ac"):
            if "values" not in st:
                ro = st["rollout"]
                ro.values = A.critic_values(tr.actor if self.shared else tr.critic, ro, self.algo)
                st["values"] = True
        elif vid == "i_pi":
            self._dpo_inputs(st, step)
        elif vid in ("t_pi", "t_ac"):
            c.update(self._train_policy(st, step))
        elif vid == "t_V":
            c.update(self._train_critic(st, step))
        else:
            raise RuntimeExecutionError(f"engine backend has no operator for vertex {vid}")
        return c

    def _dpo_inputs(self, st, step: int) -> None:
        if "rollout" in st:
            return
        torch, A, w = self.torch, self.A, self.run.workload
        g = torch.Generator().manual_seed(self.run.data.data_seed * 7919 + step)
        pr = torch.randint(3, self.vocab, (w.batch_size, w.context_length), generator=g, dtype=torch.int32).repeat_interleave(2, 0)
        rs = torch.randint(3, self.vocab, (2 * w.batch_size, w.generation_length), generator=g, dtype=torch.int32)
        sl = slice(self.rank * 2 * (w.batch_size // self.world), (self.rank + 1) * 2 * (w.batch_size // self.world))
        p, r = pr[sl].to(self.device), rs[sl].to(self.device)
        N, T = r.shape
        st["rollout"] = A.Rollout(p, [w.context_length] * N, r, [T] * N, torch.zeros((N, T), device=self.device),
                                  torch.ones((N, T), device=self.device))

    def _global(self, x: float) -> float:
        return self.trainer._global_sum(x)

    def _train_policy(self, st, step: int) -> Dict[str, Any]:
        tr, A = self.trainer, self.A
        ro = st["rollout"]
        if self.family == "pipeline_train":
            # every stage needs every microbatch: the ranks' rollouts (with reference log-probs and scores) are gathered,
            # the update runs 1F1B over the global batch, then the stages' weights go back to the replicated layout
            glob = tr.gather_rollout(ro)
            A.grpo_advantages(glob, self.run.workload.samples_per_prompt)
            st["denom"] = float(glob.n_response_tokens())
            steps = 0
            for part in self._minibatches(glob, step, ranks=1):
                m = tr.train_policy(part, st["denom"] if part is glob else float(part.n_response_tokens()))
                steps += 1
            received = tr.publish()
            m["grad_norm"] = tr.opt.grad_norm()
            out = {k: float(v) for k, v in tr._read(m).items()}
            out.update(train_tokens=int(sum(ro.total_lens())) * self.run.algorithm.epochs, optimizer_steps=steps,
                       pipeline_stages=self.world, pipeline_p2p_calls=tr.runner.p2p_calls, layout_switch_bytes=received)
            return out
        if self.algo_name == "dpo":
            tr.policy.zero_grad()
            m = A.dpo_train_step(tr.policy, ro, st["ref_seq"], self.algo, n_pairs_global=int(self._global(ro.n // 2)))
            tr.opt.step()
            m["grad_norm"] = tr.opt.grad_norm()
        else:
            if self.algo_name == "grpo":
                A.grpo_advantages(ro, self.run.workload.samples_per_prompt)
                opt = tr.opt
            else:
                if "targets" not in st:
                    A.ppo_targets(ro, self.algo)
                    st["targets"] = True
                opt = tr.opt_actor
            st["denom"] = self._global(ro.n_response_tokens())
            steps = 0
            for part in self._minibatches(ro, step):       # epochs x minibatches, one optimizer step each
                denom = st["denom"] if part is ro else self._global(part.n_response_tokens())
                tr.actor.zero_grad()
                m = A.policy_train_step(tr.actor, part, self.algo, denom_tokens=denom,
                                        **({"value_model_shared": True} if self.shared else {}))
                opt.step()
                steps += 1
            m["grad_norm"] = opt.grad_norm()
            out = {k: float(v) for k, v in tr._read(m).items()}
            out.update(train_tokens=int(sum(ro.total_lens())) * self.run.algorithm.epochs, optimizer_steps=steps)
            return out
        out = {k: float(v) for k, v in tr._read(m).items()}
        out.update(train_tokens=int(sum(ro.total_lens())), optimizer_steps=1)
        return out

    def _minibatches(self, ro, step: int, ranks: Optional[int] = None):
        """The rollout parts of the update epochs (``algorithm.epochs``, ``algorithm.minibatch_size`` sequences of
        the GLOBAL batch per optimizer step; every rank cuts its own rows the same way). One epoch without a
        minibatch size is the rollout itself."""
        a = self.run.algorithm
        if a.epochs == 1 and not a.minibatch_size:
            return [ro]
        from .data import minibatch_indices
        local = None if not a.minibatch_size else max(1, int(a.minibatch_size) // (ranks or self.world))
        return [ro.subset(rows) for rows in minibatch_indices(ro.n, local, a.epochs, seed=a.seed + step)]

    def _train_critic(self, st, step: int = 0) -> Dict[str, Any]:
        tr, A = self.trainer, self.A
        ro = st["rollout"]
        if "targets" not in st:
            A.ppo_targets(ro, self.algo)
            st["targets"] = True
        denom_all = st.get("denom") or self._global(ro.n_response_tokens())
        steps = 0
        for part in self._minibatches(ro, step):
            denom = denom_all if part is ro else self._global(part.n_response_tokens())
            tr.critic.zero_grad()
            m = A.critic_train_step(tr.critic, part, self.algo, denom_tokens=denom)
            tr.opt_critic.step()
            steps += 1
        m["critic_grad_norm"] = tr.opt_critic.grad_norm()
        out = {k: float(v) for k, v in tr._read(m).items()}
        out.update(train_tokens=int(sum(ro.total_lens())) * self.run.algorithm.epochs, optimizer_steps=steps)
        return out

    # ------------------------------------------------------------------ executor interface
    async def execute(self, node, context) -> NodeExecutionResult:
        await asyncio.sleep(0)
        from ..ops import _lib
        from ..ops import kernels as K
        step = node_step(node)
        name = model_name(node.model)
        c: Dict[str, Any] = {"kind": node.kind.value, "rank": self.rank}
        weights: List[WeightVersion] = []
        if node.kind is ExecNodeType.OP:
            n0 = _lib.launch_count()
            c.update(self._run_op(node))
            K.check_status()
            c["kernel_launches"] = _lib.launch_count() - n0
            c["peak_memory_bytes"] = int(self.torch.cuda.max_memory_allocated(self.device))
            en = node.exec_node
            if en.n_seqs is not None:
                c.update(partial_n_seqs=int(en.n_seqs), phase_forced_completions=0)
                part = split_part_index(node.node_id)
                if part is not None:
                    c["artifact_part"] = part
            if self.family == "disaggregated" and getattr(self, "_leave_together", False):
                # Last training vertex of the run. The trainers push the final weights into the generation ranks' memory:
                # a generation rank (long done) first waits on the host for that version, then all ranks meet, so that
                # no process leaves while a peer's kernel may still write into its buffers.
                import torch.distributed as dist
                self._leave_together = False
                eng = self.async_engine
                if eng.is_gen and not eng.weights.ready(int(step or 0), float(self.run.runtime.node_timeout_s)):
                    raise RuntimeExecutionError(f"final weight version {step} did not arrive")
                self.torch.cuda.synchronize()
                dist.barrier()
            if self.family == "disaggregated":
                if node.role == "TRAIN" and name is not None and self.async_engine.is_train:
                    self.latest[name] = int(step or 0)
                    c["produced_weight"] = {"model": name, "version": self.latest[name], "shadow": self.tau > 0}
                    weights.append(WeightVersion(name, self.latest[name], tuple(node.parallelism or (1, 1, 1))))
                for s in [s for s in self.steps if s < (step or 0) - self.tau - 1]:
                    del self.steps[s]
            elif name in ("actor", "critic", "ac_share") and node.role in ("GEN", "INF") and step is not None:
                c.update(weight_version=self.latest.get(name, 0), model=name, shadow=False)
            if self.family != "disaggregated" and node.role == "TRAIN" and name is not None:
                self.latest[name] = self.latest.get(name, 0) + 1
                c["produced_weight"] = {"model": name, "version": self.latest[name], "shadow": False}
                weights.append(WeightVersion(name, self.latest[name], tuple(node.parallelism or (1, 1, 1))))
                done = [s for s in self.steps if s < (step or 0)]
                for s in done:           # rollouts of closed steps are dead
                    del self.steps[s]
        elif (node.kind is ExecNodeType.RESHARD and self.family == "tp_generation" and name in ("actor", "ac_share")
              and getattr(self.trainer, "gen_tp", False)):
            # publication edge t_pi -> g_pi: the updated replicated weights are re-sliced into this rank's shards of the
            # tensor-parallel generation layout (strided device copies, timed on the device)
            gm = self.trainer.gen_model
            before = gm.refreshes
            gm.refresh()
            K.check_status()
            c.update(payload_in_bytes=node.payload_in_bytes, transferred_bytes=int(gm.shard.numel() * 2), transport="layout_switch",
                     label=node.label, reshard_us=float(gm.last_reshard_us or 0.0), layout_switches=gm.refreshes - before)
        else:
            c.update(payload_in_bytes=node.payload_in_bytes, transferred_bytes=0, transport="in_place", label=node.label)
        ref = ContainerRef(f"{node.node_id}:output", step or 0, split_part_index(node.node_id), producer=node.node_id)
        context.store.put(ref)
        return NodeExecutionResult(node.node_id, "ok", c, (ref,), tuple(weights))

    # ------------------------------------------------------------------ checkpoints
    def _trainables(self):
        if self.family == "disaggregated":
            return {}          # weights and optimizer state live on the training ranks only; no checkpoint is taken in this family
        tr = self.trainer
        if self.algo_name == "dpo":
            return {"actor": (tr.policy, tr.opt)}
        if self.algo_name == "grpo":
            return {"actor": (tr.actor, tr.opt)}
        out = {"ac_share" if self.shared else "actor": (tr.actor, tr.opt_actor)}
        if tr.critic is not None:
            out["critic"] = (tr.critic, tr.opt_critic)
        return out

    def save_checkpoint(self, step: int, path, kind: str) -> Dict[str, Any]:
        torch = self.torch
        torch.cuda.synchronize()
        total_bytes = files = 0
        for name, (model, opt) in self._trainables().items():
            d = Path(path) / name
            n = model.layout.total
            tensors = {"adam.master": opt.master, "adam.m": opt.m, "adam.v": opt.v}
            ranges = {k: (opt.shard_off, opt.shard_off + opt.shard_n, n) for k in tensors}
            if self.rank == 0:
                tensors["weights"] = model.w[:n]
            part = ckpt.save_flat_shards(d, self.rank, self.world, tensors, ranges=ranges,
                                         extra={"optimizer_step": opt.step_count, "version": self.latest.get(name, 0)})
            total_bytes += part["file"]["bytes"]
            files += 1
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        if self.rank == 0:
            for name in self._trainables():
                ckpt.finalize_worker_meta(Path(path) / name, self.world, extra={"step": step, "kind": kind})
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        return {"workers": sorted(self._trainables()), "bytes": total_bytes, "files": files}

    def restore_checkpoint(self, step: int, path) -> None:
        for name, (model, opt) in self._trainables().items():
            d = Path(path) / name
            n = model.layout.total
            model.w[:n].copy_(ckpt.load_tensor(d, "weights").to(self.device))
            lo, hi = opt.shard_off, opt.shard_off + opt.shard_n
            opt.master.copy_(ckpt.load_flat_range(d, "adam.master", lo, hi).to(self.device))
            opt.m.copy_(ckpt.load_flat_range(d, "adam.m", lo, hi).to(self.device))
            opt.v.copy_(ckpt.load_flat_range(d, "adam.v", lo, hi).to(self.device))
            meta = json.loads((d / "meta.json").read_text())
            opt.step_count = int(meta["ranks"][0]["extra"]["optimizer_step"])
            self.latest[name] = int(meta["ranks"][0]["extra"]["version"])
        if hasattr(self.trainer, "ref") and self.algo_name != "dpo":
            pass    # the frozen reference never changes; nothing to restore
        self.steps.clear()
        self.torch.cuda.synchronize()


def make_engine_handler_factory(compiled):
    """One engine (models, optimizer state, KV arena) lives for the whole run; replays reuse it and
    restore its state from the checkpoint instead of rebuilding it."""
    holder: Dict[str, EngineOperationHandler] = {}

    def make(attempt: int):
        if "h" not in holder:
            holder["h"] = EngineOperationHandler(compiled, attempt)
        holder["h"].attempt = attempt
        return holder["h"]

    return make
