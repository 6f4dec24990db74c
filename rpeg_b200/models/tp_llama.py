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
