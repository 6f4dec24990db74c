"""Tensor-parallel forward of the Llama-family decoder (inference: reference log-probs, reward and value
passes) built from the fused linear layers of ``parallel.tp``.

Activations travel between layers in the sequence-parallel layout (every rank holds ``T / world`` token rows);
inside a layer the Megatron pattern applies:

    x_sp -RMSNorm-> (all-gather + GEMM: QKV for this rank's heads) -RoPE-> attention over ALL tokens, local heads
         -> (GEMM + reduce-scatter: output projection) -> + residual (sequence-parallel rows)
         -RMSNorm-> (all-gather + GEMM: gate/up slice) -SwiGLU-> (GEMM + reduce-scatter: down projection) -> + residual

so each layer launches exactly two all-gather+GEMM kernels and two GEMM+reduce-scatter kernels and no NCCL call.
The weights are this rank's tensor-parallel shards, cut out of the replicated training weights by the reshard
rules (``parallel.reshard.tp_pieces``): q/k/v heads, gate and up rows, o/down columns. The LM head is vocabulary
parallel; token log-probs combine the per-shard max / sum-exp / target logit with three small all-reduces.
Packed variable-length sequences are padded to a multiple of ``128 * world`` tokens (padding rows form one extra
sequence that nobody reads). Reference: Megatron GPTModel with ``tensor_model_parallel_size = tp`` as built in
RPEG/runtime/workers/megatron_worker.py:676-715, vocab-parallel logits gathered in :1657-1760.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import kernels as K
from ..parallel.reshard import param_shapes, tp_pieces
from ..parallel.tp import ROW_BLOCK, ColumnParallelLinear, RowParallelLinear
from .llama import LlamaConfig, LlamaModel


class TPLlamaForward:
    def __init__(self, model: LlamaModel, max_tokens: int, group=None):
        """``model`` holds the full (replicated) weights; this object keeps the rank's shards and the fused layers.
        ``max_tokens`` bounds the packed token count of one call (rounded up to ``128 * world``)."""
        self.full = model
        self.cfg = cfg = model.cfg
        self.device = model.device
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        w = self.world
        if cfg.n_heads % w or cfg.n_kv_heads % w or cfg.d_ff % w or cfg.vocab % w:
            raise ValueError(f"heads ({cfg.n_heads}/{cfg.n_kv_heads}), d_ff ({cfg.d_ff}) and vocab ({cfg.vocab}) must divide by tp={w}")
        if cfg.qk_norm:
            raise NotImplementedError("tensor-parallel forward without QK-norm only")
        unit = ROW_BLOCK * w
        self.max_tokens = (max_tokens + unit - 1) // unit * unit
        self.h_loc, self.hkv_loc = cfg.n_heads // w, cfg.n_kv_heads // w
        # Layers run one after the other, so all column-parallel layers (input width d) share one pair of input
        # buffers and all row-parallel layers (output width d) one staging / output set; only the weights differ.
        shapes = param_shapes(cfg)
        names = [f"l{i}.{n}" for i in range(cfg.n_layers) for n in ("wqkv", "wo", "w_gate_up", "w_down")] + (["lm_head"] if cfg.lm_head else [])
        self.shards = {n: self._shard(n, shapes) for n in names}
        self.col = ColumnParallelLinear(self.shards["l0.wqkv"], self.max_tokens, self.device, group)
        self.row = RowParallelLinear(self.shards["l0.wo"], self.max_tokens, self.device, group)
        self.vocab0 = self.rank * (cfg.vocab // w)

    def _shard(self, name: str, shapes) -> torch.Tensor:
        """This rank's tensor-parallel pieces of ``name`` stacked in order (q|k|v heads, gate|up rows, column slice)."""
        full = self.full.p[name]
        parts = [full[r0:r1, c0:c1] for r0, r1, c0, c1 in tp_pieces(self.cfg, name, shapes[name], self.world, self.rank)]
        return (torch.cat(parts, 0) if len(parts) > 1 else parts[0]).contiguous()

    def refresh_weights(self) -> None:
        """Re-cut the shards after the replicated weights changed (an optimizer step)."""
        shapes = param_shapes(self.cfg)
        for name, t in self.shards.items():
            t.copy_(self._shard(name, shapes))

    # ------------------------------------------------------------------ forward
    def _pad(self, tokens, pos, cu_seqlens, max_seqlen):
        T = tokens.numel()
        unit = ROW_BLOCK * self.world
        Tp = (T + unit - 1) // unit * unit
        if Tp > self.max_tokens:
            raise ValueError(f"{T} tokens exceed max_tokens={self.max_tokens}")
        if Tp != T:
            pad = Tp - T
            tokens = torch.cat([tokens, torch.zeros(pad, dtype=tokens.dtype, device=tokens.device)])
            pos = torch.cat([pos, torch.arange(pad, dtype=pos.dtype, device=pos.device) % self.cfg.max_pos])
            cu_seqlens = torch.cat([cu_seqlens, torch.tensor([Tp], dtype=cu_seqlens.dtype, device=cu_seqlens.device)])
            max_seqlen = max(max_seqlen, min(pad, self.cfg.max_pos))
        return tokens, pos, cu_seqlens, max_seqlen, T, Tp

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor, pos: torch.Tensor, cu_seqlens: torch.Tensor, max_seqlen: int) -> Tuple[torch.Tensor, int]:
        """Returns this rank's rows ``[Tp / world, d]`` of the final normalised hidden states and the padded
        token count ``Tp`` (global row ``g`` lives on rank ``g // (Tp / world)``)."""
        cfg, p = self.cfg, self.full.p
        tokens, pos, cu, max_seqlen, T, Tp = self._pad(tokens, pos, cu_seqlens, int(max_seqlen))
        per = Tp // self.world
        sl = slice(self.rank * per, (self.rank + 1) * per)
        h = K.embed_fwd(tokens[sl].contiguous(), p["embed"])                 # sequence-parallel rows
        qw, kvw = self.h_loc * cfg.head_dim, self.hkv_loc * cfg.head_dim
        for i in range(cfg.n_layers):
            x, _, _ = K.rmsnorm_fwd(h, p[f"l{i}.attn_norm"], cfg.rms_eps)
            col = self.col.use_weight(self.shards[f"l{i}.wqkv"])
            col.input_rows(Tp).copy_(x)
            qkv = col.forward(Tp)                                            # [Tp, (h_loc + 2 hkv_loc) * hd]
            K.rope_(qkv, pos, self.full.cos_t, self.full.sin_t, 0, self.h_loc, cfg.head_dim)
            K.rope_(qkv, pos, self.full.cos_t, self.full.sin_t, qw, self.hkv_loc, cfg.head_dim)
            attn, _ = K.flash_attn_fwd(qkv, 0, qw, qw + kvw, cu, max_seqlen, self.h_loc, self.hkv_loc, cfg.head_dim)
            o = self.row.use_weight(self.shards[f"l{i}.wo"]).forward(attn)   # [per, d], reduce-scattered rows
            x2, _, h = K.rmsnorm_fwd(o, p[f"l{i}.mlp_norm"], cfg.rms_eps, residual=h, want_sum=True)
            col = self.col.use_weight(self.shards[f"l{i}.w_gate_up"])
            col.input_rows(Tp).copy_(x2)
            act = K.swiglu_fwd(col.forward(Tp))                              # [Tp, d_ff / world]
            dn = self.row.use_weight(self.shards[f"l{i}.w_down"]).forward(act)
            h = K.add_bf16(h, dn)
        xf, _, _ = K.rmsnorm_fwd(h, p["final_norm"], cfg.rms_eps)
        return xf, Tp

    @torch.no_grad()
    def token_logprobs(self, tokens: torch.Tensor, pos: torch.Tensor, cu_seqlens: torch.Tensor, max_seqlen: int,
                       targets: torch.Tensor, temperature: float = 1.0) -> torch.Tensor:
        """``log p(targets[t] | prefix)`` for every packed token ``t`` (``[T]`` fp32, identical on all ranks)."""
        if "lm_head" not in self.shards:
            raise RuntimeError("model has no LM head")
        T = tokens.numel()
        xf, Tp = self.forward(tokens, pos, cu_seqlens, max_seqlen)
        col = self.col.use_weight(self.shards["lm_head"])
        col.input_rows(Tp).copy_(xf)
        logits = col.forward(Tp)[:T].float() / temperature                    # [T, V / world]
        tl = targets.long() - self.vocab0
        mine = (tl >= 0) & (tl < logits.shape[1])
        m = logits.max(-1).values
        if self.world > 1:
            dist.all_reduce(m, op=dist.ReduceOp.MAX, group=self.group)
        s = (logits - m[:, None]).exp().sum(-1)
        tgt = torch.where(mine, logits.gather(1, tl.clamp(0, logits.shape[1] - 1)[:, None])[:, 0], torch.zeros_like(m))
        if self.world > 1:
            dist.all_reduce(s, group=self.group)
            dist.all_reduce(tgt, group=self.group)
        return tgt - (m + s.log())

    def close(self) -> None:
        self.col.close()
        self.row.close()


class _FlatLayout:
    def __init__(self, total: int):
        self.total = total


class TPLlamaTrain:
    """Tensor-parallel TRAINING of the decoder: forward, backward and optimizer state on this rank's shards, with
    every linear layer - in both directions - running through the two fused kernels.

    Per layer (activations between layers are sequence parallel, ``[T / world, d]``):

        forward    RMSNorm -> all-gather + GEMM (QKV, local heads) -> RoPE -> attention -> GEMM + reduce-scatter (O)
                   -> RMSNorm(+residual) -> all-gather + GEMM (gate/up slice) -> SwiGLU -> GEMM + reduce-scatter (down)
        backward   the mirror image: the gradient of a reduce-scattered output is all-gathered INTO the GEMM that
                   multiplies it with the weight shard (all-gather + GEMM), and the partial input gradients of a
                   column-parallel layer are summed across ranks BY the GEMM that produces them (GEMM + reduce-scatter).
                   Weight gradients are local GEMMs on operands the fused kernels already gathered.

    The kernels take the weight as ``[out, in]`` with ``in`` contiguous, so the backward uses transposed copies of
    the shards (rebuilt after every optimizer step). The layer is recomputed from its sequence-parallel input in the
    backward pass (only layer inputs are kept). Parameters live in one flat bf16 buffer, replicated ones (embedding,
    norms) first, then the shards; gradients in one flat fp32 buffer of the same layout. Replicated parameters see
    only this rank's token rows, so their gradients are summed over the tensor-parallel group before the optimizer
    step; the global gradient norm adds the shards' squared norms over the group and the replicated part once.
    Reference: Megatron tensor parallelism as configured in RPEG/runtime/workers/megatron_worker.py:676-715, with
    the gradient all-reduces of :878-881 replaced by the fused collectives inside the GEMMs.
    """

    SHARDED = ("wqkv", "wo", "w_gate_up", "w_down")

    def __init__(self, full: LlamaModel, max_tokens: int, group=None):
        cfg = full.cfg
        if cfg.qk_norm or cfg.tie_embeddings or not cfg.lm_head:
            raise NotImplementedError("tensor-parallel training: untied LM head, no QK-norm")
        self.cfg, self.device, self.group = cfg, full.device, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        w = self.world
        if cfg.n_heads % w or cfg.n_kv_heads % w or cfg.d_ff % w or cfg.vocab % (8 * w):
            raise ValueError("heads, d_ff and vocab / 8 must divide by the tensor-parallel degree")
        self.h_loc, self.hkv_loc = cfg.n_heads // w, cfg.n_kv_heads // w
        unit = ROW_BLOCK * w
        self.max_tokens = (max_tokens + unit - 1) // unit * unit
        shapes = param_shapes(cfg)
        rep = ["embed", "final_norm"] + [f"l{i}.{n}" for i in range(cfg.n_layers) for n in ("attn_norm", "mlp_norm")]
        shd = [f"l{i}.{n}" for i in range(cfg.n_layers) for n in self.SHARDED] + ["lm_head"]
        self.entries = {}
        off = 0

        def add(name, shape):
            nonlocal off
            self.entries[name] = (off, tuple(shape))
            off += (math.prod(shape) + 63) // 64 * 64

        for n in rep:
            add(n, shapes[n])
        self.n_replicated = off
        pieces = {n: tp_pieces(cfg, n, shapes[n], w, self.rank) for n in shd}
        for n in shd:
            rows = sum(r1 - r0 for r0, r1, _, _ in pieces[n])
            cols = pieces[n][0][3] - pieces[n][0][2]
            add(n, (rows, cols))
        self.layout = _FlatLayout(off)
        self.w = torch.zeros(off, dtype=torch.bfloat16, device=self.device)
        self.g = torch.zeros(off, dtype=torch.float32, device=self.device)
        view = lambda flat, n: flat[self.entries[n][0]: self.entries[n][0] + math.prod(self.entries[n][1])].view(*self.entries[n][1])
        self.p = {n: view(self.w, n) for n in self.entries}
        self.gp = {n: view(self.g, n) for n in self.entries}
        for n in rep:
            self.p[n].copy_(full.p[n])
        for n in shd:
            parts = [full.p[n][r0:r1, c0:c1] for r0, r1, c0, c1 in pieces[n]]
            self.p[n].copy_(torch.cat(parts, 0) if len(parts) > 1 else parts[0])
        self.pieces = pieces
        self.wt = {n: torch.empty((self.entries[n][1][1], self.entries[n][1][0]), dtype=torch.bfloat16, device=self.device) for n in shd}
        self.refresh_transposes()
        self.cos_t, self.sin_t = full.cos_t, full.sin_t
        self.col = ColumnParallelLinear(self.p["l0.wqkv"], self.max_tokens, self.device, group)
        self.row = RowParallelLinear(self.p["l0.wo"], self.max_tokens, self.device, group)
        self.vocab0 = self.rank * (cfg.vocab // w)

    # ------------------------------------------------------------------ parameters
    def refresh_transposes(self) -> None:
        """``[in, out]`` copies of the shards for the backward GEMMs (call after every optimizer step)."""
        for n, t in self.wt.items():
            t.copy_(self.p[n].t())

    def zero_grad(self) -> None:
        self.g.zero_()

    def sync_replicated_grads(self) -> None:
        """Sum the gradients of the replicated parameters over the tensor-parallel group (each rank saw its rows)."""
        if self.world > 1:
            dist.all_reduce(self.g[: self.n_replicated], group=self.group)

    # ------------------------------------------------------------------ fused linear helpers
    def _col(self, weight: torch.Tensor, x_sp: torch.Tensor, Tp: int) -> torch.Tensor:
        c = self.col.use_weight(weight)
        c.input_rows(Tp).copy_(x_sp)
        return c.forward(Tp)

    def _row(self, weight: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        return self.row.use_weight(weight).forward(x)

    # ------------------------------------------------------------------ one layer
    def _layer_fwd(self, i: int, h: torch.Tensor, pos, cu, max_seqlen: int, Tp: int, keep: bool):
        cfg, p = self.cfg, self.p
        qw, kvw = self.h_loc * cfg.head_dim, self.hkv_loc * cfg.head_dim
        x1, rstd1, _ = K.rmsnorm_fwd(h, p[f"l{i}.attn_norm"], cfg.rms_eps)
        qkv = self._col(p[f"l{i}.wqkv"], x1, Tp)
        X1 = self.col.gathered(Tp).clone() if keep else None
        K.rope_(qkv, pos, self.cos_t, self.sin_t, 0, self.h_loc, cfg.head_dim)
        K.rope_(qkv, pos, self.cos_t, self.sin_t, qw, self.hkv_loc, cfg.head_dim)
        attn, lse = K.flash_attn_fwd(qkv, 0, qw, qw + kvw, cu, max_seqlen, self.h_loc, self.hkv_loc, cfg.head_dim)
        o = self._row(p[f"l{i}.wo"], attn)
        x2, rstd2, h1 = K.rmsnorm_fwd(o, p[f"l{i}.mlp_norm"], cfg.rms_eps, residual=h, want_sum=True)
        gu = self._col(p[f"l{i}.w_gate_up"], x2, Tp)
        X2 = self.col.gathered(Tp).clone() if keep else None
        act = K.swiglu_fwd(gu)
        dn = self._row(p[f"l{i}.w_down"], act)
        h_out = K.add_bf16(h1, dn)
        saved = dict(rstd1=rstd1, X1=X1, qkv=qkv, attn=attn, lse=lse, h1=h1, rstd2=rstd2, X2=X2, gu=gu, act=act) if keep else None
        return h_out, saved

    def _layer_bwd(self, i: int, h_in: torch.Tensor, d_out: torch.Tensor, pos, cu, max_seqlen: int, Tp: int) -> torch.Tensor:
        cfg, p, g, wt = self.cfg, self.p, self.gp, self.wt
        qw, kvw = self.h_loc * cfg.head_dim, self.hkv_loc * cfg.head_dim
        _, s = self._layer_fwd(i, h_in, pos, cu, max_seqlen, Tp, keep=True)           # recompute from the layer input
        # down projection (row parallel): all-gather d_out into the GEMM with the weight shard
        d_act = self._col(wt[f"l{i}.w_down"], d_out, Tp)                               # [Tp, f / w]
        K.gemm(self.col.gathered(Tp), s["act"], trans_a=True, trans_b=True, out=g[f"l{i}.w_down"], accumulate=True)
        d_gu = K.swiglu_bwd(s["gu"], d_act)
        # gate/up projection (column parallel): partial input gradients summed by the GEMM's reduce-scatter
        d_x2 = self._row(wt[f"l{i}.w_gate_up"], d_gu)                                  # [Tp / w, d]
        K.gemm(d_gu, s["X2"], trans_a=True, trans_b=True, out=g[f"l{i}.w_gate_up"], accumulate=True)
        d_h1 = K.rmsnorm_bwd(d_x2, s["h1"], p[f"l{i}.mlp_norm"], s["rstd2"], g[f"l{i}.mlp_norm"], dres_in=d_out)
        # output projection (row parallel)
        d_attn = self._col(wt[f"l{i}.wo"], d_h1, Tp)                                   # [Tp, q / w]
        K.gemm(self.col.gathered(Tp), s["attn"], trans_a=True, trans_b=True, out=g[f"l{i}.wo"], accumulate=True)
        d_qkv = K.flash_attn_bwd(s["qkv"], 0, qw, qw + kvw, s["attn"], d_attn, s["lse"], cu, max_seqlen, self.h_loc, self.hkv_loc,
                                 cfg.head_dim)
        K.rope_(d_qkv, pos, self.cos_t, self.sin_t, 0, self.h_loc, cfg.head_dim, backward=True)
        K.rope_(d_qkv, pos, self.cos_t, self.sin_t, qw, self.hkv_loc, cfg.head_dim, backward=True)
        # QKV projection (column parallel)
        d_x1 = self._row(wt[f"l{i}.wqkv"], d_qkv)
        K.gemm(d_qkv, s["X1"], trans_a=True, trans_b=True, out=g[f"l{i}.wqkv"], accumulate=True)
        return K.rmsnorm_bwd(d_x1, h_in, p[f"l{i}.attn_norm"], s["rstd1"], g[f"l{i}.attn_norm"], dres_in=d_h1)

    # ------------------------------------------------------------------ one microbatch
    def forward_backward(self, tokens: torch.Tensor, pos: torch.Tensor, cu_seqlens: torch.Tensor, max_seqlen: int,
                         targets: torch.Tensor, coef_fn, temperature: float = 1.0) -> torch.Tensor:
        """``targets [T]`` int32 with -1 on rows without a loss term; ``coef_fn(logp [T]) -> d loss / d logp [T]``.
        Accumulates the gradients of this microbatch and returns ``logp [T]`` (identical on all ranks)."""
        cfg, p, g = self.cfg, self.p, self.gp
        T = tokens.numel()
        unit = ROW_BLOCK * self.world
        Tp = (T + unit - 1) // unit * unit
        if Tp > self.max_tokens:
            raise ValueError(f"{T} tokens exceed max_tokens={self.max_tokens}")
        if Tp != T:
            pad = Tp - T
            dev = tokens.device
            tokens = torch.cat([tokens, torch.zeros(pad, dtype=tokens.dtype, device=dev)])
            pos = torch.cat([pos, torch.arange(pad, dtype=pos.dtype, device=dev) % cfg.max_pos])
            cu_seqlens = torch.cat([cu_seqlens, torch.tensor([Tp], dtype=cu_seqlens.dtype, device=dev)])
            max_seqlen = max(int(max_seqlen), min(pad, cfg.max_pos))
            targets = torch.cat([targets, torch.full((pad,), -1, dtype=targets.dtype, device=dev)])
        per = Tp // self.world
        sl = slice(self.rank * per, (self.rank + 1) * per)
        my_tokens = tokens[sl].contiguous()
        h = K.embed_fwd(my_tokens, p["embed"])
        inputs = []
        for i in range(cfg.n_layers):
            inputs.append(h)
            h, _ = self._layer_fwd(i, h, pos, cu_seqlens, int(max_seqlen), Tp, keep=False)
        xf, rstd_f, _ = K.rmsnorm_fwd(h, p["final_norm"], cfg.rms_eps)
        # vocabulary-parallel head: local logits, global log-sum-exp and target logit, gradient in place
        logits = self._col(p["lm_head"], xf, Tp)                                       # [Tp, V / w]
        xf_full = self.col.gathered(Tp)
        tl = targets.to(torch.int32) - self.vocab0
        mine = (targets >= 0) & (tl >= 0) & (tl < logits.shape[1])
        tl = torch.where(mine, tl, torch.full_like(tl, -1)).contiguous()
        lp_loc, lse_loc = K.token_logprob_fwd(logits, tl, temperature)
        x_y = torch.where(mine, lp_loc + lse_loc, torch.zeros_like(lp_loc))
        if self.world > 1:
            dist.all_reduce(x_y, group=self.group)
            all_lse = torch.empty((self.world, Tp), dtype=lse_loc.dtype, device=lse_loc.device)
            dist.all_gather_into_tensor(all_lse.view(-1), lse_loc.contiguous(), group=self.group)
            lse = torch.logsumexp(all_lse, dim=0)
        else:
            lse = lse_loc
        logp = torch.where(targets >= 0, x_y - lse, torch.zeros_like(lse))
        coef = coef_fn(logp[:T])
        if Tp != T:
            coef = torch.cat([coef, torch.zeros(Tp - T, dtype=coef.dtype, device=coef.device)])
        K.token_logprob_bwd_(logits, tl, lse.contiguous(), coef.contiguous().float(), temperature)
        d_xf = self._row(self.wt["lm_head"], logits)                                    # [Tp / w, d]
        K.gemm(logits, xf_full, trans_a=True, trans_b=True, out=g["lm_head"], accumulate=True)
        d_h = K.rmsnorm_bwd(d_xf, h, p["final_norm"], rstd_f, g["final_norm"])
        for i in reversed(range(cfg.n_layers)):
            d_h = self._layer_bwd(i, inputs.pop(), d_h, pos, cu_seqlens, int(max_seqlen), Tp)
        K.embed_bwd(my_tokens, d_h, g["embed"])
        return logp[:T]

    def close(self) -> None:
        self.col.close()
        self.row.close()


class TPAdamW:
    """AdamW on fp32 master copies of a ``TPLlamaTrain``'s flat parameter buffer. The clip coefficient uses the
    global norm: squared norms of the shards summed over the tensor-parallel group, the replicated part once."""

    def __init__(self, model: TPLlamaTrain, *, lr: float = 1e-6, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                 max_grad_norm: float = 1.0):
        self.model, self.lr, self.betas, self.eps, self.wd, self.max_grad_norm = model, lr, betas, eps, weight_decay, max_grad_norm
        self.step_count = 0
        dev = model.device
        self.master = model.w.float()
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self._part = torch.zeros(1, dtype=torch.float32, device=dev)

    def grad_norm(self) -> torch.Tensor:
        return self.sumsq.sqrt()

    def step(self, sync_replicated: bool = True) -> None:
        """``sync_replicated=False`` when the caller already summed the replicated parameters' gradients."""
        m = self.model
        self.step_count += 1
        if sync_replicated:
            m.sync_replicated_grads()
        self._part.zero_()
        K.sumsq(m.g[m.n_replicated:], self._part)
        if m.world > 1:
            dist.all_reduce(self._part, group=m.group)
        self.sumsq.zero_()
        K.sumsq(m.g[: m.n_replicated], self.sumsq)
        self.sumsq.add_(self._part)
        b1, b2 = self.betas
        K.adamw_(self.master, self.m, self.v, m.g, m.w, lr=self.lr, beta1=b1, beta2=b2, eps=self.eps, wd=self.wd,
                 step=self.step_count, grad_scale=1.0, sumsq=self.sumsq, max_norm=self.max_grad_norm)
        m.refresh_transposes()
