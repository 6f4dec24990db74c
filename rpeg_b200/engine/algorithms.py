"""PPO / GRPO / DPO operators on one GPU's share of a batch, built from the native kernels.

The verbs match the reference's worker operation surface (RPEG/runtime/semantic.py:495-537 and the
dispatch in RPEG/runtime/semantic_worker.py:425-621) so the runtime handler maps graph vertices
one to one: ``generate`` (g_pi/g_ac), ``reference_logprobs`` (i_ref), ``reward_scores`` (i_R),
``critic_values`` (i_V/i_ac), ``policy_train_step`` (t_pi, PPO and GRPO), ``critic_train_step``
(t_V), ``actor_critic_train_step`` (t_ac), ``dpo_train_step``.

Loss definitions are the reference's (RPEG/runtime/workers/megatron_worker.py:4264-4274, 4361-4417,
4650; RPEG/runtime/ppo_math.py:14-92): clipped ratio objective normalised by the global response
token count, ``kl_coef * (logp - logp_ref)`` for GRPO, masked value MSE, DPO over interleaved
(chosen, rejected) rows.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ..models.llama import LlamaModel
from ..ops import kernels as K
from .batching import PackedBatch, pack_rows, split_microbatches


@dataclass
class Rollout:
    """Everything one iteration carries between operators (all tensors on the device)."""
    prompt_ids: torch.Tensor                 # [N, S] int32
    prompt_lens: List[int]
    resp_ids: torch.Tensor                   # [N, T] int32
    resp_lens: List[int]
    old_logp: torch.Tensor                   # [N, T] fp32, from sampling
    mask: torch.Tensor                       # [N, T] fp32 response mask
    ref_logp: Optional[torch.Tensor] = None
    values: Optional[torch.Tensor] = None
    scores: Optional[torch.Tensor] = None    # [N]
    adv: Optional[torch.Tensor] = None       # [N, T]
    returns: Optional[torch.Tensor] = None
    weight_version: int = 0

    @property
    def n(self) -> int:
        return self.resp_ids.shape[0]

    def total_lens(self) -> List[int]:
        return [p + r for p, r in zip(self.prompt_lens, self.resp_lens)]

    def n_response_tokens(self) -> int:
        return int(sum(self.resp_lens))

    def subset(self, rows: Sequence[int]) -> "Rollout":
        """The rollout restricted to ``rows`` (a minibatch of an update epoch); tensors are gathered copies."""
        idx = torch.tensor(list(rows), dtype=torch.long, device=self.resp_ids.device)
        pick = lambda t: None if t is None else t[idx].contiguous()
        return Rollout(pick(self.prompt_ids), [self.prompt_lens[i] for i in rows], pick(self.resp_ids), [self.resp_lens[i] for i in rows],
                       pick(self.old_logp), pick(self.mask), pick(self.ref_logp), pick(self.values), pick(self.scores), pick(self.adv),
                       pick(self.returns), self.weight_version)


@dataclass
class AlgoConfig:
    clip_eps: float = 0.2
    kl_coef: float = 0.0
    beta: float = 0.1            # PPO KL-reward coefficient and DPO temperature
    gamma: float = 1.0
    gae_lambda: float = 0.95
    value_coef: float = 0.5
    entropy_coef: float = 0.0    # the policy objective gets  - entropy_coef * mean token entropy  (an exploration bonus)
    normalize_advantages: bool = True
    temperature: float = 1.0
    micro_tokens: int = 16384    # packed tokens per microbatch
    head_chunk: int = 8192       # rows of logits materialised at a time


def _micro(ro: Rollout, cfg: AlgoConfig, group: int = 1) -> List[PackedBatch]:
    parts = split_microbatches(ro.total_lens(), cfg.micro_tokens, group)
    return [pack_rows(ro.prompt_ids, ro.prompt_lens, ro.resp_ids, ro.resp_lens, rows) for rows in parts]


# ---------------------------------------------------------------------------------- inference ops
@torch.no_grad()
def sequence_logprobs(model: LlamaModel, ro: Rollout, cfg: AlgoConfig, pipeline=None) -> torch.Tensor:
    """Per-token log-probs of the responses under ``model`` -> ``[N, T]`` (zeros outside the mask). With a
    ``parallel.pp.PipelineRunner`` the microbatches stream through the stages and the last stage's result is
    relayed to all of them."""
    out = torch.zeros_like(ro.old_logp)
    flat_out = out.view(-1)

    def head(mb, xf):
        flat_out[mb.flat] = model.token_logprobs(K.gather_rows(xf, mb.sel), mb.targets, cfg.head_chunk, cfg.temperature)

    if pipeline is not None:
        pipeline.run(_micro(ro, cfg), head, train=False)
        return pipeline.broadcast_from_last(out)
    for mb in _micro(ro, cfg):
        xf, _ = model.forward(mb.tokens, mb.pos, mb.cu_seqlens, mb.max_seqlen)
        head(mb, xf)
    return out


@torch.no_grad()
def reward_scores(model: LlamaModel, ro: Rollout, cfg: AlgoConfig) -> torch.Tensor:
    """Scalar head at the last token of every sequence -> ``[N]``."""
    out = torch.zeros(ro.n, dtype=torch.float32, device=model.device)
    for mb in _micro(ro, cfg):
        xf, _ = model.forward(mb.tokens, mb.pos, mb.cu_seqlens, mb.max_seqlen)
        out[torch.tensor(mb.rows, device=model.device)] = model.scalar_values(K.gather_rows(xf, mb.last))
    return out


@torch.no_grad()
def critic_values(model: LlamaModel, ro: Rollout, cfg: AlgoConfig) -> torch.Tensor:
    """Scalar head on the rows that predict each response token -> ``[N, T]``."""
    out = torch.zeros_like(ro.old_logp)
    flat_out = out.view(-1)
    for mb in _micro(ro, cfg):
        xf, _ = model.forward(mb.tokens, mb.pos, mb.cu_seqlens, mb.max_seqlen)
        flat_out[mb.flat] = model.scalar_values(K.gather_rows(xf, mb.sel))
    return out


def ppo_targets(ro: Rollout, cfg: AlgoConfig) -> None:
    """KL-shaped token rewards + GAE + returns (+ masked whitening) into ``ro.adv`` / ``ro.returns``."""
    ro.adv, ro.returns = K.gae(ro.old_logp, ro.ref_logp, ro.values, ro.mask, ro.scores, cfg.beta, cfg.gamma,
                               cfg.gae_lambda, cfg.normalize_advantages)


def grpo_advantages(ro: Rollout, samples_per_prompt: int) -> None:
    """Group-normalised sequence rewards broadcast over the response tokens."""
    a = K.group_advantage(ro.scores.contiguous(), samples_per_prompt)
    ro.adv = (a[:, None] * ro.mask).contiguous()


# ---------------------------------------------------------------------------------- training ops
def _scatter_head_grad(xf: torch.Tensor, sel: torch.Tensor, d_rows: torch.Tensor) -> torch.Tensor:
    d_xf = torch.zeros_like(xf)
    K.scatter_rows_(d_xf, sel, d_rows, overwrite=True)
    return d_xf


def make_policy_head(model: LlamaModel, ro: Rollout, cfg: AlgoConfig, denom: float, value_model_shared: bool = False):
    """``head(mb, xf) -> d_xf`` of the clipped policy objective for one microbatch (LM head forward/backward fused with
    the loss), plus the accumulators it adds its partial sums to: ``(head, acc[4], vacc[4])``. The closure is what a
    plain microbatch loop, a pipeline's last stage or a fused two-model pipeline calls on the final hidden states."""
    acc = torch.zeros(4, dtype=torch.float32, device=model.device)
    vacc = torch.zeros(4, dtype=torch.float32, device=model.device)
    old, adv, mask = ro.old_logp.view(-1), ro.adv.view(-1), ro.mask.view(-1)
    ref = ro.ref_logp.view(-1) if (ro.ref_logp is not None and cfg.kl_coef != 0.0) else None

    def head(mb, xf):
        rows = K.gather_rows(xf, mb.sel)
        o_mb, a_mb, m_mb = old[mb.flat], adv[mb.flat], mask[mb.flat]
        r_mb = ref[mb.flat] if ref is not None else None

        def coef_fn(s, e, lp):
            coef, part = K.policy_loss(lp, o_mb[s:e], None if r_mb is None else r_mb[s:e], a_mb[s:e], m_mb[s:e],
                                       cfg.clip_eps, cfg.kl_coef, 1.0 / denom)
            acc.add_(part)
            return coef

        def entropy_fn(s, e, ent):
            ecoef = m_mb[s:e] * (-cfg.entropy_coef / denom)          # d loss / d H per token
            acc[0].add_((ecoef * ent).sum())
            vacc[1].add_((m_mb[s:e] * ent).sum())
            return ecoef.contiguous()

        _, d_rows = model.lm_head_fwd_bwd(rows, mb.targets, coef_fn, cfg.head_chunk, cfg.temperature,
                                          entropy_fn=entropy_fn if cfg.entropy_coef != 0.0 else None)
        if value_model_shared:
            v = model.scalar_values(rows)
            dv, part = K.value_loss(v, ro.returns.view(-1)[mb.flat], m_mb, 1.0 / denom)
            vacc.add_(part)
            d_rows = K.add_bf16(d_rows, model.scalar_head_bwd(rows, dv * cfg.value_coef))
        return _scatter_head_grad(xf, mb.sel, d_rows)

    return head, acc, vacc


def make_critic_head(model: LlamaModel, ro: Rollout, cfg: AlgoConfig, denom: float):
    """``head(mb, xf) -> d_xf`` of the masked value loss and its accumulator ``acc[4]``."""
    acc = torch.zeros(4, dtype=torch.float32, device=model.device)
    ret, mask = ro.returns.view(-1), ro.mask.view(-1)

    def head(mb, xf):
        rows = K.gather_rows(xf, mb.sel)
        v = model.scalar_values(rows)
        dv, part = K.value_loss(v, ret[mb.flat], mask[mb.flat], 1.0 / denom)
        acc.add_(part)
        return _scatter_head_grad(xf, mb.sel, model.scalar_head_bwd(rows, dv))

    return head, acc


def policy_train_step(model: LlamaModel, ro: Rollout, cfg: AlgoConfig, *, denom_tokens: Optional[float] = None,
                      value_model_shared: bool = False, pipeline=None, on_last_backward=None) -> Dict[str, torch.Tensor]:
    """Forward + backward of the clipped policy objective over the whole rollout (gradients are
    accumulated over microbatches; the caller runs the optimizer). ``denom_tokens`` is the GLOBAL
    response-token count when the batch is sharded over data-parallel ranks. With
    ``value_model_shared`` the same trunk also fits the value head (actor-critic sharing). With a
    ``parallel.pp.PipelineRunner`` (``model`` being this rank's stage) the microbatches run in 1F1B order, the
    loss is evaluated on the last stage and the metrics are relayed to every stage."""
    denom = float(denom_tokens if denom_tokens is not None else max(1, ro.n_response_tokens()))
    head, acc, vacc = make_policy_head(model, ro, cfg, denom, value_model_shared)
    if pipeline is not None:
        pipeline.run(_micro(ro, cfg), head, train=True)
        pipeline.broadcast_from_last(acc)
        pipeline.broadcast_from_last(vacc)
    else:
        mbs = list(_micro(ro, cfg))
        for idx, mb in enumerate(mbs):
            xf, ctx = model.forward(mb.tokens, mb.pos, mb.cu_seqlens, mb.max_seqlen, keep=True)
            d_xf = head(mb, xf)
            # ``on_last_backward(layer)``: the gradients of the layers from ``layer`` up are final once the last
            # microbatch's backward has passed it (``parallel.dp.DPContext.overlap_hook`` reduces them right away)
            model.grad_hook = on_last_backward if idx + 1 == len(mbs) else None
            try:
                model.backward(ctx, d_xf)
            finally:
                model.grad_hook = None
    return {"loss": acc[0], "kl_sum": acc[1], "clipped": acc[2], "approx_kl_sum": acc[3], "value_loss": vacc[0],
            "entropy_sum": vacc[1]}


def critic_train_step(model: LlamaModel, ro: Rollout, cfg: AlgoConfig, *, denom_tokens: Optional[float] = None,
                      pipeline=None) -> Dict[str, torch.Tensor]:
    denom = float(denom_tokens if denom_tokens is not None else max(1, ro.n_response_tokens()))
    head, acc = make_critic_head(model, ro, cfg, denom)
    if pipeline is not None:
        pipeline.run(_micro(ro, cfg), head, train=True)
        pipeline.broadcast_from_last(acc)
    else:
        for mb in _micro(ro, cfg):
            xf, ctx = model.forward(mb.tokens, mb.pos, mb.cu_seqlens, mb.max_seqlen, keep=True)
            model.backward(ctx, head(mb, xf))
    return {"value_loss": acc[0]}


def policy_train_step_tp(tp_model, ro: Rollout, cfg: AlgoConfig, *, denom_tokens: Optional[float] = None) -> Dict[str, torch.Tensor]:
    """The clipped policy objective on a tensor-parallel model (``models.tp_llama.TPLlamaTrain``): every rank of
    the tensor-parallel group calls this with the SAME rollout; linear layers run through the fused all-gather /
    reduce-scatter GEMMs in both directions and the vocabulary-parallel head closes the loss on all ranks at once."""
    denom = float(denom_tokens if denom_tokens is not None else max(1, ro.n_response_tokens()))
    dev = ro.resp_ids.device
    acc = torch.zeros(4, dtype=torch.float32, device=dev)
    old, adv, mask = ro.old_logp.view(-1), ro.adv.view(-1), ro.mask.view(-1)
    ref = ro.ref_logp.view(-1) if (ro.ref_logp is not None and cfg.kl_coef != 0.0) else None
    for mb in _micro(ro, cfg):
        T = int(mb.tokens.numel())
        sel = mb.sel.long()
        targets = torch.full((T,), -1, dtype=torch.int32, device=dev)
        targets[sel] = mb.targets.to(torch.int32)
        o_mb, a_mb, m_mb = old[mb.flat].contiguous(), adv[mb.flat].contiguous(), mask[mb.flat].contiguous()
        r_mb = ref[mb.flat].contiguous() if ref is not None else None

        def coef_fn(logp_full):
            coef_sel, part = K.policy_loss(logp_full[sel].contiguous(), o_mb, r_mb, a_mb, m_mb, cfg.clip_eps, cfg.kl_coef, 1.0 / denom)
            acc.add_(part)
            out = torch.zeros(T, dtype=torch.float32, device=dev)
            out[sel] = coef_sel
            return out

        tp_model.forward_backward(mb.tokens, mb.pos, mb.cu_seqlens, mb.max_seqlen, targets, coef_fn, cfg.temperature)
    return {"loss": acc[0], "kl_sum": acc[1], "clipped": acc[2], "approx_kl_sum": acc[3]}


def fused_actor_critic_train_step(actor_stage: LlamaModel, critic_stage: LlamaModel, ro: Rollout, cfg: AlgoConfig, executor, *,
                                  denom_tokens: Optional[float] = None) -> Dict[str, torch.Tensor]:
    """PPO's two training vertices as ONE interleaved pipeline step (``parallel.fused_pp.FusedPipelineExecutor``):
    the actor's stages run in device order, the critic's in reverse order on the same GPUs, and every device
    follows the precomputed instruction stream that mixes the two models' forward and backward microtasks.
    The actor's loss lives on the last device, the critic's on the first; metrics are relayed to all ranks."""
    denom = float(denom_tokens if denom_tokens is not None else max(1, ro.n_response_tokens()))
    a_head, acc, _ = make_policy_head(actor_stage, ro, cfg, denom)
    c_head, cacc = make_critic_head(critic_stage, ro, cfg, denom)
    mbs = _micro(ro, cfg)
    executor.run({"actor": mbs, "critic": mbs}, {"actor": a_head, "critic": c_head})
    executor.broadcast_from_last("actor", acc)
    executor.broadcast_from_last("critic", cacc)
    return {"loss": acc[0], "kl_sum": acc[1], "clipped": acc[2], "approx_kl_sum": acc[3], "value_loss": cacc[0]}


def dpo_train_step(model: LlamaModel, ro: Rollout, ref_seq_logp: torch.Tensor, cfg: AlgoConfig, *,
                   n_pairs_global: Optional[int] = None) -> Dict[str, torch.Tensor]:
    """Rows are interleaved (chosen, rejected). ``ref_seq_logp [N]`` are the frozen model's masked
    sequence log-probs. A pair never straddles microbatches, so every microbatch closes its own loss:
    its log-probs are reduced per sequence, the pair loss yields ``d loss / d logp`` per token, and a
    second pass over the LM head (logits recomputed chunk by chunk) turns that into gradients."""
    P_local = ro.n // 2
    P = int(n_pairs_global if n_pairs_global is not None else P_local)
    acc = torch.zeros(4, dtype=torch.float32, device=model.device)
    T = ro.resp_ids.shape[1]
    for mb in _micro(ro, cfg, group=2):
        xf, ctx = model.forward(mb.tokens, mb.pos, mb.cu_seqlens, mb.max_seqlen, keep=True)
        rows = K.gather_rows(xf, mb.sel)
        with torch.no_grad():
            lp = model.token_logprobs(rows, mb.targets, cfg.head_chunk)
        n_mb = len(mb.rows)
        lp_mat = torch.zeros((n_mb, T), dtype=torch.float32, device=model.device)
        row_t = torch.tensor(mb.rows, device=model.device)
        local_flat = mb.flat - (row_t[0] * T)          # rows of a microbatch are consecutive
        lp_mat.view(-1)[local_flat] = lp
        m_mat = ro.mask[row_t]
        pi_seq = K.masked_rowsum(lp_mat, m_mat.contiguous())
        seq_coef, part = K.dpo_loss(pi_seq, ref_seq_logp[row_t].contiguous(), cfg.beta)
        scale = (n_mb // 2) / P                        # kernel normalises by local pairs
        acc[0] += part[0] * scale
        acc[1:3] += part[1:3]
        coef_tok = (K.expand_seq_coef(seq_coef, m_mat.contiguous()) * scale).view(-1)[local_flat].contiguous()
        _, d_rows = model.lm_head_fwd_bwd(rows, mb.targets, lambda s, e, _lp: coef_tok[s:e], cfg.head_chunk)
        model.backward(ctx, _scatter_head_grad(xf, mb.sel, d_rows))
    return {"loss": acc[0], "n_correct": acc[1], "margin_sum": acc[2]}
