"""Llama-style dense decoder (RMSNorm, RoPE, SwiGLU, causal attention) executed entirely by the
native sm_100a kernels, with an explicit forward and backward instead of autograd.

Why explicit: the training step is a fixed chain (norm -> QKV GEMM -> RoPE -> flash attention ->
out-proj -> norm -> gate/up GEMM -> SwiGLU -> down GEMM), so the backward is written once against
the kernels, weight gradients accumulate straight into one flat fp32 buffer from the wgrad GEMM
epilogue, and the memory policy (recompute a layer from its saved input, or keep its activations)
is a flag rather than a tracing decision.

Parameters live in ONE flat bf16 buffer (and gradients in one flat fp32 buffer); every tensor is a
view. Data-parallel optimizer sharding, the fused reduce-scatter + Adam + all-gather kernels, weight
publication to generation replicas and checkpoints all address that flat space by offset.

Roles the reference builds with megatron-core's GPTModel plus auxiliary heads
(RPEG/runtime/workers/megatron_worker.py:642-843): actor / reference (LM head), critic / reward
(scalar head ``Linear(d, 1)`` on the final hidden state), shared actor-critic (both heads).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from ..ops import kernels as K


@dataclass(frozen=True)
class LlamaConfig:
    n_layers: int = 32
    d_model: int = 4096
    d_ff: int = 11008
    n_heads: int = 32
    n_kv_heads: int = 32
    head_dim: int = 128
    vocab: int = 32000
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_pos: int = 4096
    lm_head: bool = True
    scalar_head: bool = False
    qk_norm: bool = False               # per-head RMSNorm on queries and keys before RoPE (Qwen3)
    tie_embeddings: bool = False        # the LM head shares the embedding matrix
    rope_scaling_factor: float = 1.0    # llama3 long-context frequency scaling
    family: str = "llama"

    @property
    def q_width(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.n_kv_heads * self.head_dim

    @property
    def qkv_width(self) -> int:
        return self.q_width + 2 * self.kv_width

    def n_params(self) -> int:
        return ParamLayout(self).total

    @classmethod
    def llama7b(cls, **kw) -> "LlamaConfig":
        return cls(32, 4096, 11008, 32, 32, 128, 32000, **kw)

    @classmethod
    def llama13b(cls, **kw) -> "LlamaConfig":
        return cls(40, 5120, 13824, 40, 40, 128, 32000, **kw)

    @classmethod
    def qwen3_8b(cls, **kw) -> "LlamaConfig":
        base = dict(n_layers=36, d_model=4096, d_ff=12288, n_heads=32, n_kv_heads=8, head_dim=128, vocab=151936, rms_eps=1e-6,
                    rope_theta=1e6, qk_norm=True, family="qwen3")
        base.update(kw)
        return cls(**base)

    @classmethod
    def tiny(cls, **kw) -> "LlamaConfig":
        base = dict(n_layers=2, d_model=256, d_ff=512, n_heads=2, n_kv_heads=2, head_dim=128, vocab=512, max_pos=512)
        base.update(kw)
        return cls(**base)


_ALIGN = 64  # elements; keeps every tensor 128-byte aligned in the flat buffers


def stage_layers(n_layers: int, stage: Optional[Tuple[int, int]]) -> Tuple[int, int]:
    """Layer range ``[lo, hi)`` of pipeline stage ``(index, n_stages)``: contiguous blocks, the first
    ``n_layers % n_stages`` stages one layer longer (the rule of RPEG/runtime/reshard.py:60-98)."""
    if stage is None:
        return 0, n_layers
    idx, n = stage
    if not 0 <= idx < n or n > n_layers:
        raise ValueError(f"bad pipeline stage {stage} for {n_layers} layers")
    per, extra = divmod(n_layers, n)
    lo = idx * per + min(idx, extra)
    return lo, lo + per + (1 if idx < extra else 0)


class ParamLayout:
    """Name -> (offset, shape) of every parameter inside the flat buffer."""

    def __init__(self, cfg: LlamaConfig, stage: Optional[Tuple[int, int]] = None):
        """``stage = (index, n_stages)`` keeps only that pipeline stage's parameters: its block of layers, the
        embedding on the first stage, the final norm and the heads on the last (a tied LM head keeps its own
        copy of the embedding matrix on the last stage when the two stages differ)."""
        self.cfg = cfg
        self.entries: Dict[str, Tuple[int, Tuple[int, ...]]] = {}
        self.layer_lo, self.layer_hi = stage_layers(cfg.n_layers, stage)
        self.first = stage is None or stage[0] == 0
        self.last = stage is None or stage[0] == stage[1] - 1
        off = 0

        def add(name: str, *shape: int) -> None:
            nonlocal off
            self.entries[name] = (off, tuple(shape))
            n = math.prod(shape)
            off += (n + _ALIGN - 1) // _ALIGN * _ALIGN

        d, f = cfg.d_model, cfg.d_ff
        tied_head = cfg.lm_head and cfg.tie_embeddings
        if self.first or (self.last and tied_head):
            add("embed", cfg.vocab, d)
        for i in range(self.layer_lo, self.layer_hi):
            add(f"l{i}.attn_norm", d)
            add(f"l{i}.wqkv", cfg.qkv_width, d)
            if cfg.qk_norm:
                add(f"l{i}.q_norm", cfg.head_dim)
                add(f"l{i}.k_norm", cfg.head_dim)
            add(f"l{i}.wo", d, cfg.q_width)
            add(f"l{i}.mlp_norm", d)
            add(f"l{i}.w_gate_up", 2 * f, d)
            add(f"l{i}.w_down", d, f)
        if self.last:
            add("final_norm", d)
            if cfg.lm_head and not cfg.tie_embeddings:
                add("lm_head", cfg.vocab, d)
            if cfg.scalar_head:
                add("scalar_head.w", d)
                add("scalar_head.b", 8)  # element 0 is the bias; padded to a 16-byte slot
        self.total = off

    def view(self, flat: torch.Tensor, name: str) -> torch.Tensor:
        off, shape = self.entries[name]
        return flat[off:off + math.prod(shape)].view(*shape)


@dataclass
class _LayerCtx:
    h_in: torch.Tensor                       # layer input (always kept)
    saved: Optional[dict] = None             # intermediate activations when not recomputing


@dataclass
class _FwdCtx:
    tokens: torch.Tensor
    pos: torch.Tensor
    cu_seqlens: torch.Tensor
    max_seqlen: int
    layers: List[_LayerCtx] = field(default_factory=list)
    h_last: Optional[torch.Tensor] = None    # input of the final norm
    rstd_f: Optional[torch.Tensor] = None


class LlamaModel:
    """Weights + kernels for one model instance on one GPU."""

    def __init__(self, cfg: LlamaConfig, device, *, trainable: bool = False, recompute: str = "full",
                 weights: Optional[torch.Tensor] = None, grads: Optional[torch.Tensor] = None, seed: int = 0,
                 stage: Optional[Tuple[int, int]] = None):
        """``stage = (index, n_stages)`` builds one pipeline stage: ``forward`` then takes the previous stage's
        hidden states (``h_in``) unless it is the first, and returns raw hidden states unless it is the last."""
        if cfg.head_dim != 128:
            raise ValueError("the attention kernels are specialised for head_dim = 128")
        if recompute not in ("full", "none"):
            raise ValueError("recompute must be 'full' or 'none'")
        # with recompute == "full": the activations of the LAST `keep_layers` layers are kept all the same (as much of the
        # second forward pass is skipped as the memory left on the GPU pays for; the backward pass frees those first)
        self.keep_layers = 0
        self.cfg = cfg
        self.device = torch.device(device)
        self.layout = ParamLayout(cfg, stage)
        self.stage = stage
        self.layer_lo, self.layer_hi = self.layout.layer_lo, self.layout.layer_hi
        self.is_first, self.is_last = self.layout.first, self.layout.last
        self.recompute = recompute
        self.w = weights if weights is not None else torch.empty(self.layout.total, dtype=torch.bfloat16, device=self.device)
        if self.w.numel() < self.layout.total:
            raise ValueError("weight buffer smaller than the parameter layout")
        self.g = None
        if trainable:
            self.g = grads if grads is not None else torch.zeros(self.layout.total, dtype=torch.float32, device=self.device)
        self.p = {name: self.layout.view(self.w, name) for name in self.layout.entries}
        self.gp = {name: self.layout.view(self.g, name) for name in self.layout.entries} if self.g is not None else {}
        if cfg.lm_head and cfg.tie_embeddings and self.is_last:      # one matrix, two uses: both gradients accumulate into it
            self.p["lm_head"] = self.p["embed"]
            if self.g is not None:
                self.gp["lm_head"] = self.gp["embed"]
        self.cos_t, self.sin_t = K.rope_tables(cfg.max_pos, cfg.head_dim, cfg.rope_theta, self.device, cfg.rope_scaling_factor)
        self._ws: Optional[torch.Tensor] = None  # split-K scratch for decode GEMMs
        # One-shot weight-version gate (flags, min_version, timeout_s): the next full-sequence forward hands it to
        # its first GEMM, which then loads no weight tile before the version is complete (weights that other GPUs
        # are pushing into this model's buffer).
        self.weight_gate = None
        # ``grad_hook(i)`` is called by ``backward`` right after layer ``i``'s gradient kernels are queued (the final
        # norm and the heads are complete by then): the data-parallel step starts reducing finished layers under the rest
        # of the backward pass (set for the LAST microbatch of a step only: earlier ones still accumulate)
        self.grad_hook = None
        if weights is None:
            self.init_weights(seed)

    # ------------------------------------------------------------------ init / utilities
    def init_weights(self, seed: int = 0) -> None:
        gen = torch.Generator(device=self.device)
        gen.manual_seed(seed)
        self.w.zero_()
        for name, (off, shape) in self.layout.entries.items():
            v = self.p[name]
            if name.endswith("norm"):
                v.fill_(1.0)
            elif name == "scalar_head.b":
                v.zero_()
            else:
                fan_in = shape[-1]
                std = 1.0 / math.sqrt(fan_in) if name.startswith("scalar_head") else 0.02
                v.copy_(torch.randn(shape, generator=gen, device=self.device, dtype=torch.float32) * std)

    def zero_grad(self) -> None:
        if self.g is not None:
            self.g.zero_()

    def load_flat(self, other: "LlamaModel") -> None:
        n = min(self.layout.total, other.layout.total)
        self.w[:n].copy_(other.w[:n])

    def kv_columns(self):
        """(first K column, first V column, KV heads) of the heads this model keeps in a generator's KV cache,
        inside the QKV activation a full-sequence forward hands to ``kv_sink``."""
        return self.cfg.q_width, self.cfg.q_width + self.cfg.kv_width, self.cfg.n_kv_heads

    def _workspace(self) -> torch.Tensor:
        if self._ws is None:
            self._ws = torch.empty(32 * 1024 * 1024, dtype=torch.float32, device=self.device)
        return self._ws

    def _lin(self, x: torch.Tensor, w: torch.Tensor, decode: bool = False) -> torch.Tensor:
        return K.gemm(x, w, workspace=self._workspace() if decode else None)

    def _qk_norm(self, i: int, qkv: torch.Tensor, keep_pre: bool):
        """Per-head RMSNorm of the query and key heads in place. Returns what backward needs (the
        pre-norm q|k columns and the two rstd tensors) or None."""
        cfg, p = self.cfg, self.p
        pre = qkv[:, : cfg.q_width + cfg.kv_width].clone() if keep_pre else None
        rq = K.headnorm_fwd_(qkv, 0, cfg.n_heads, cfg.head_dim, p[f"l{i}.q_norm"], cfg.rms_eps, want_rstd=keep_pre)
        rk = K.headnorm_fwd_(qkv, cfg.q_width, cfg.n_kv_heads, cfg.head_dim, p[f"l{i}.k_norm"], cfg.rms_eps, want_rstd=keep_pre)
        return (pre, rq, rk) if keep_pre else None

    # ------------------------------------------------------------------ full-sequence forward
    def _layer_fwd(self, i: int, res: torch.Tensor, delta: Optional[torch.Tensor], ctx: _FwdCtx, keep: bool, gate=None):
        """One decoder layer on packed tokens. Input is the residual stream as ``res (+ delta)``;
        returns ``(h1, dn)`` with the layer output being ``h1 + dn`` (the add is fused into the next
        RMSNorm)."""
        cfg, p = self.cfg, self.p
        keep_acts = keep and (self.recompute == "none" or i >= self.layer_hi - self.keep_layers)
        if delta is None:
            h = res
            x, rstd1, _ = K.rmsnorm_fwd(h, p[f"l{i}.attn_norm"], cfg.rms_eps)
        else:
            x, rstd1, h = K.rmsnorm_fwd(delta, p[f"l{i}.attn_norm"], cfg.rms_eps, residual=res, want_sum=True)
        qkv = K.gemm(x, p[f"l{i}.wqkv"], gate=gate)
        qkn = self._qk_norm(i, qkv, keep_acts) if cfg.qk_norm else None
        K.rope_(qkv, ctx.pos, self.cos_t, self.sin_t, 0, cfg.n_heads, cfg.head_dim)
        K.rope_(qkv, ctx.pos, self.cos_t, self.sin_t, cfg.q_width, cfg.n_kv_heads, cfg.head_dim)
        attn, lse = K.flash_attn_fwd(qkv, 0, cfg.q_width, cfg.q_width + cfg.kv_width, ctx.cu_seqlens, ctx.max_seqlen,
                                     cfg.n_heads, cfg.n_kv_heads, cfg.head_dim)
        o = K.gemm(attn, p[f"l{i}.wo"])
        x2, rstd2, h1 = K.rmsnorm_fwd(o, p[f"l{i}.mlp_norm"], cfg.rms_eps, residual=h, want_sum=True)
        if keep_acts or cfg.d_ff % 128:
            gu = K.gemm(x2, p[f"l{i}.w_gate_up"])          # the backward pass wants the pre-activation
            act = K.swiglu_fwd(gu)
        else:
            gu = None
            act = K.gemm_swiglu(x2, p[f"l{i}.w_gate_up"])  # activation in the GEMM epilogue: [T, 2f] never exists
        dn = K.gemm(act, p[f"l{i}.w_down"])
        if keep:
            saved = None
            if keep_acts:
                saved = dict(x=x, rstd1=rstd1, qkv=qkv, attn=attn, lse=lse, h1=h1, x2=x2, rstd2=rstd2, gu=gu, act=act, qkn=qkn)
            ctx.layers.append(_LayerCtx(h_in=h, saved=saved))
        return h1, dn, qkv

    def forward(self, tokens: torch.Tensor, pos: torch.Tensor, cu_seqlens: torch.Tensor, max_seqlen: int,
                keep: bool = False, kv_sink=None, h_in: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Optional[_FwdCtx]]:
        """Packed causal forward. Returns the final normalised hidden states ``[T, d]`` and, with
        ``keep=True``, the context ``backward`` needs. ``kv_sink(layer, qkv)`` receives each layer's
        rotated QKV (generation prefill stores K/V into the paged cache through it). A pipeline stage
        other than the first starts from ``h_in [T, d]``; one other than the last returns the raw
        residual stream for the next stage."""
        cfg = self.cfg
        ctx = _FwdCtx(tokens, pos, cu_seqlens, int(max_seqlen))
        if self.is_first:
            res, delta = K.embed_fwd(tokens, self.p["embed"]), None
        else:
            if h_in is None:
                raise ValueError("a pipeline stage after the first needs h_in")
            res, delta = h_in, None
        gate, self.weight_gate = self.weight_gate, None
        for i in range(self.layer_lo, self.layer_hi):
            res, delta, qkv = self._layer_fwd(i, res, delta, ctx, keep, gate if i == self.layer_lo else None)
            if kv_sink is not None:
                kv_sink(i, qkv)
        if not self.is_last:
            return K.add_bf16(res, delta), (ctx if keep else None)
        xf, rstd_f, h_last = K.rmsnorm_fwd(delta, self.p["final_norm"], cfg.rms_eps, residual=res, want_sum=True)
        if keep:
            ctx.h_last, ctx.rstd_f = h_last, rstd_f
        return xf, (ctx if keep else None)

    # ------------------------------------------------------------------ backward
    def _layer_bwd(self, i: int, lc: _LayerCtx, d_out: torch.Tensor, ctx: _FwdCtx) -> torch.Tensor:
        cfg, p, g = self.cfg, self.p, self.gp
        h = lc.h_in
        s = lc.saved
        if s is None:  # recompute the layer from its input
            x, rstd1, _ = K.rmsnorm_fwd(h, p[f"l{i}.attn_norm"], cfg.rms_eps)
            qkv = K.gemm(x, p[f"l{i}.wqkv"])
            qkn = self._qk_norm(i, qkv, True) if cfg.qk_norm else None
            K.rope_(qkv, ctx.pos, self.cos_t, self.sin_t, 0, cfg.n_heads, cfg.head_dim)
            K.rope_(qkv, ctx.pos, self.cos_t, self.sin_t, cfg.q_width, cfg.n_kv_heads, cfg.head_dim)
            attn, lse = K.flash_attn_fwd(qkv, 0, cfg.q_width, cfg.q_width + cfg.kv_width, ctx.cu_seqlens,
                                         ctx.max_seqlen, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim)
            o = K.gemm(attn, p[f"l{i}.wo"])
            x2, rstd2, h1 = K.rmsnorm_fwd(o, p[f"l{i}.mlp_norm"], cfg.rms_eps, residual=h, want_sum=True)
            del o
            gu = K.gemm(x2, p[f"l{i}.w_gate_up"])
            act = K.swiglu_fwd(gu)
        else:
            x, rstd1, qkv, attn, lse = s["x"], s["rstd1"], s["qkv"], s["attn"], s["lse"]
            h1, x2, rstd2, gu, act = s["h1"], s["x2"], s["rstd2"], s["gu"], s["act"]
            qkn = s.get("qkn")
        # MLP
        d_act = K.gemm(d_out, p[f"l{i}.w_down"], trans_b=True)
        K.gemm(d_out, act, trans_a=True, trans_b=True, out=g[f"l{i}.w_down"], accumulate=True)
        del act
        d_gu = K.swiglu_bwd(gu, d_act)
        del gu, d_act
        d_x2 = K.gemm(d_gu, p[f"l{i}.w_gate_up"], trans_b=True)
        K.gemm(d_gu, x2, trans_a=True, trans_b=True, out=g[f"l{i}.w_gate_up"], accumulate=True)
        del d_gu, x2
        d_h1 = K.rmsnorm_bwd(d_x2, h1, p[f"l{i}.mlp_norm"], rstd2, g[f"l{i}.mlp_norm"], dres_in=d_out)
        del d_x2, h1
        # attention
        d_attn = K.gemm(d_h1, p[f"l{i}.wo"], trans_b=True)
        K.gemm(d_h1, attn, trans_a=True, trans_b=True, out=g[f"l{i}.wo"], accumulate=True)
        d_qkv = K.flash_attn_bwd(qkv, 0, cfg.q_width, cfg.q_width + cfg.kv_width, attn, d_attn, lse, ctx.cu_seqlens,
                                 ctx.max_seqlen, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim)
        del d_attn, attn, qkv
        K.rope_(d_qkv, ctx.pos, self.cos_t, self.sin_t, 0, cfg.n_heads, cfg.head_dim, backward=True)
        K.rope_(d_qkv, ctx.pos, self.cos_t, self.sin_t, cfg.q_width, cfg.n_kv_heads, cfg.head_dim, backward=True)
        if cfg.qk_norm:
            pre, rq, rk = qkn
            for name, col0, nh, r in (("q_norm", 0, cfg.n_heads, rq), ("k_norm", cfg.q_width, cfg.n_kv_heads, rk)):
                dw = torch.zeros(cfg.head_dim, dtype=torch.float32, device=self.device)
                K.headnorm_bwd_(d_qkv, pre, col0, nh, cfg.head_dim, p[f"l{i}.{name}"], r, dw)
                g[f"l{i}.{name}"].add_(dw)
            del pre, rq, rk, qkn
        d_x = K.gemm(d_qkv, p[f"l{i}.wqkv"], trans_b=True)
        K.gemm(d_qkv, x, trans_a=True, trans_b=True, out=g[f"l{i}.wqkv"], accumulate=True)
        del d_qkv, x
        return K.rmsnorm_bwd(d_x, h, p[f"l{i}.attn_norm"], rstd1, g[f"l{i}.attn_norm"], dres_in=d_h1)

    def backward(self, ctx: _FwdCtx, d_xf: torch.Tensor) -> Optional[torch.Tensor]:
        """Accumulate parameter gradients given ``d loss / d xf`` (``xf`` = output of ``forward``). A pipeline
        stage other than the first returns the gradient of its input for the previous stage."""
        if self.g is None:
            raise RuntimeError("model was built without gradient storage (trainable=False)")
        if self.is_last:
            d_h = K.rmsnorm_bwd(d_xf, ctx.h_last, self.p["final_norm"], ctx.rstd_f, self.gp["final_norm"])
            ctx.h_last = None
        else:
            d_h = d_xf
        for i in reversed(range(self.layer_lo, self.layer_hi)):
            lc = ctx.layers.pop()
            d_h = self._layer_bwd(i, lc, d_h, ctx)
            if self.grad_hook is not None:
                self.grad_hook(i)
        if not self.is_first:
            return d_h
        K.embed_bwd(ctx.tokens, d_h, self.gp["embed"])
        return None

    # ------------------------------------------------------------------ heads
    def token_logprobs(self, xf_rows: torch.Tensor, targets: torch.Tensor, chunk: int = 8192,
                       temperature: float = 1.0) -> torch.Tensor:
        """``log p(target)`` for the given hidden rows, never holding more than ``chunk`` rows of logits."""
        out = torch.empty(xf_rows.shape[0], dtype=torch.float32, device=self.device)
        for s in range(0, xf_rows.shape[0], chunk):
            e = min(xf_rows.shape[0], s + chunk)
            logits = K.gemm(xf_rows[s:e], self.p["lm_head"])
            lp, _ = K.token_logprob_fwd(logits, targets[s:e], temperature)
            out[s:e] = lp
        return out

    def lm_head_fwd_bwd(self, xf_rows: torch.Tensor, targets: torch.Tensor, coef_fn, chunk: int = 8192,
                        temperature: float = 1.0, entropy_fn=None) -> Tuple[torch.Tensor, torch.Tensor]:
        """LM head forward and backward in one pass per chunk.

        ``coef_fn(start, end, logp_chunk) -> d loss / d logp`` for rows ``[start, end)`` (any loss
        that is separable per token can be evaluated right after the chunk's log-probs exist, so
        the logits are produced once, turned into their own gradient in place and consumed by the
        dgrad / wgrad GEMMs). ``entropy_fn(start, end, entropy_chunk) -> d loss / d entropy`` adds a term in the
        per-token entropy of the softmax (an entropy bonus): the chunk's entropies are computed from the same logits
        and both gradients are written in one pass. Returns ``(logp [n], d_xf_rows [n, d])``."""
        n, d = xf_rows.shape
        logp = torch.empty(n, dtype=torch.float32, device=self.device)
        d_x = torch.empty((n, d), dtype=torch.bfloat16, device=self.device)
        for s in range(0, n, chunk):
            e = min(n, s + chunk)
            xs = xf_rows[s:e]
            logits = K.gemm(xs, self.p["lm_head"])
            lp, lse = K.token_logprob_fwd(logits, targets[s:e], temperature)
            logp[s:e] = lp
            coef = coef_fn(s, e, lp)
            if entropy_fn is None:
                K.token_logprob_bwd_(logits, targets[s:e], lse, coef, temperature)
            else:
                ent = K.token_entropy(logits, lse, temperature)
                K.token_logprob_entropy_bwd_(logits, targets[s:e], lse, coef, ent, entropy_fn(s, e, ent), temperature)
            K.gemm(logits, self.p["lm_head"], trans_b=True, out=d_x[s:e])
            K.gemm(logits, xs, trans_a=True, trans_b=True, out=self.gp["lm_head"], accumulate=True)
        return logp, d_x

    def scalar_values(self, xf_rows: torch.Tensor) -> torch.Tensor:
        return K.head_gemv(xf_rows, self.p["scalar_head.w"], self.p["scalar_head.b"].float()[:1])

    def scalar_head_bwd(self, xf_rows: torch.Tensor, dout: torch.Tensor) -> torch.Tensor:
        gw = torch.zeros(self.cfg.d_model, dtype=torch.float32, device=self.device)
        gb = torch.zeros(1, dtype=torch.float32, device=self.device)
        d_x = K.head_gemv_bwd(xf_rows, self.p["scalar_head.w"], dout, gw, gb)
        self.gp["scalar_head.w"].add_(gw)
        self.gp["scalar_head.b"][:1].add_(gb)
        return d_x

    # ------------------------------------------------------------------ decode (one token per slot)
    def decode_step(self, token: torch.Tensor, pos: torch.Tensor, slot_ids: torch.Tensor, seq_len: torch.Tensor,
                    page_table: torch.Tensor, kcache: List[torch.Tensor], vcache: List[torch.Tensor],
                    nsplit: int = 1, groups=None) -> torch.Tensor:
        """One autoregressive step for ``B`` slots: appends this token's K/V to the paged cache at
        ``pos`` and attends over ``seq_len`` cached keys. Returns the final normalised hidden ``[B, d]``.
        All GEMMs have ``M = B <= 256`` and run split-K so every SM streams a slice of the weights.
        ``groups`` (see ``ops.kernels.paged_decode_attn``) names the rows that share their first KV pages."""
        cfg, p = self.cfg, self.p
        ws = self._workspace()
        scale = 1.0 / math.sqrt(cfg.head_dim)
        if cfg.qk_norm:
            return self._decode_step_unfused(token, pos, slot_ids, seq_len, page_table, kcache, vcache, nsplit)
        # Every GEMM leaves its split-K partials in the workspace and the next kernel adds them up while it
        # loads them (one stream, so a consumer always runs before the next GEMM reuses the workspace).
        B = token.shape[0]
        h = K.embed_fwd(token, p["embed"])
        x, _, _ = K.rmsnorm_fwd(h, p["l0.attn_norm"], cfg.rms_eps)
        qkv = torch.empty((B, cfg.qkv_width), dtype=torch.bfloat16, device=self.device)
        for i in range(cfg.n_layers):
            parts = K.gemm_partials(x, p[f"l{i}.wqkv"], ws)
            K.rope_kv_append_partials_(parts, qkv, 0, cfg.q_width, cfg.q_width + cfg.kv_width, slot_ids, pos, self.cos_t,
                                       self.sin_t, page_table, kcache[i], vcache[i], cfg.n_heads, cfg.n_kv_heads, cfg.head_dim)
            attn = K.paged_decode_attn(qkv, 0, kcache[i], vcache[i], page_table, seq_len, cfg.n_heads, cfg.n_kv_heads,
                                       cfg.head_dim, scale, nsplit=nsplit, groups=groups)
            parts = K.gemm_partials(attn, p[f"l{i}.wo"], ws)
            x2, h1 = K.rmsnorm_fwd_partials(parts, p[f"l{i}.mlp_norm"], cfg.rms_eps, residual=h, want_sum=True)
            parts = K.gemm_partials(x2, p[f"l{i}.w_gate_up"], ws)
            act = K.swiglu_fwd_partials(parts)
            parts = K.gemm_partials(act, p[f"l{i}.w_down"], ws)
            last = i + 1 == cfg.n_layers
            x, h = K.rmsnorm_fwd_partials(parts, p["final_norm"] if last else p[f"l{i + 1}.attn_norm"], cfg.rms_eps, residual=h1,
                                          want_sum=not last)
        return x

    def _decode_step_unfused(self, token, pos, slot_ids, seq_len, page_table, kcache, vcache, nsplit: int = 1) -> torch.Tensor:
        """The same step with reduced GEMM outputs (needed when q and k are normalised per head before RoPE)."""
        cfg, p = self.cfg, self.p
        ws = self._workspace()
        scale = 1.0 / math.sqrt(cfg.head_dim)
        res, delta = K.embed_fwd(token, p["embed"]), None
        for i in range(cfg.n_layers):
            if delta is None:
                h = res
                x, _, _ = K.rmsnorm_fwd(h, p[f"l{i}.attn_norm"], cfg.rms_eps)
            else:
                x, _, h = K.rmsnorm_fwd(delta, p[f"l{i}.attn_norm"], cfg.rms_eps, residual=res, want_sum=True)
            qkv = K.gemm(x, p[f"l{i}.wqkv"], workspace=ws)
            if cfg.qk_norm:
                self._qk_norm(i, qkv, False)
            K.rope_kv_append_(qkv, 0, cfg.q_width, cfg.q_width + cfg.kv_width, slot_ids, pos, self.cos_t, self.sin_t,
                              page_table, kcache[i], vcache[i], cfg.n_heads, cfg.n_kv_heads, cfg.head_dim)
            attn = K.paged_decode_attn(qkv, 0, kcache[i], vcache[i], page_table, seq_len, cfg.n_heads, cfg.n_kv_heads,
                                       cfg.head_dim, scale, nsplit=nsplit)
            o = K.gemm(attn, p[f"l{i}.wo"], workspace=ws)
            x2, _, h1 = K.rmsnorm_fwd(o, p[f"l{i}.mlp_norm"], cfg.rms_eps, residual=h, want_sum=True)
            gu = K.gemm(x2, p[f"l{i}.w_gate_up"], workspace=ws)
            act = K.swiglu_fwd(gu)
            delta = K.gemm(act, p[f"l{i}.w_down"], workspace=ws)
            res = h1
        xf, _, _ = K.rmsnorm_fwd(delta, p["final_norm"], cfg.rms_eps, residual=res)
        return xf

    def lm_logits(self, xf: torch.Tensor, decode: bool = False) -> torch.Tensor:
        return K.gemm(xf, self.p["lm_head"], workspace=self._workspace() if decode else None)
