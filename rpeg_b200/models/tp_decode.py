"""Tensor-parallel view of a ``LlamaModel`` for generation.

Training keeps the whole bf16 model on every GPU (data parallel, sharded optimizer). Decoding with that layout makes
every GPU stream ALL weights for its share of the rows at every step, which is what caps generation once the batch
per GPU is small. ``TPDecodeModel`` re-slices the local copy into the tensor-parallel layout of the generation
vertex, ``(dp, pp, tp) = (1, 1, world)``:

    wqkv      rows of this rank's query heads | key heads | value heads            [3 * d / tp, d]
    wo        columns of this rank's heads                                         [d, d / tp]
    gate/up   this rank's gate rows | up rows                                      [2 * f / tp, d]
    down      this rank's columns                                                  [d, f / tp]
    LM head   this rank's vocabulary rows (a view, no copy)                         [V / tp, d]

so each GPU streams 1/tp of the weights for all rows, holds the KV cache of its own heads only, and the two
partial sums per layer are combined by ``TPCommRegion.allreduce_rmsnorm`` (reduce-scatter + residual + RMSNorm +
all-gather in one kernel over NVLink). ``refresh()`` is the layout switch after an optimizer step: strided local
copies, timed on the device (``last_reshard_us``). Prompts are prefilled with the whole local model (replicated),
each rank keeping the K/V of its heads.

Everything a rank computes outside its shard (norms, sampling, bookkeeping) is replicated bit for bit, so the
ranks stay in lock step without exchanging control messages. Reference: tensor-parallel generation of the Megatron
worker (RPEG/runtime/workers/megatron_worker.py:2301-3107), the layout switch between a training and a generation
layout (RPEG/runtime/semantic_worker.py:5503-5872) and the shard rules of RPEG/runtime/reshard.py:16-98.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import kernels as K
from ..ops._lib import check, lib
from ..parallel.tp_comm import TPCommRegion
from .llama import LlamaModel


class TPDecodeModel:
    def __init__(self, full: LlamaModel, group=None, max_batch: int = 256, comm_mode: Optional[str] = None,
                 one_shot_rows: Optional[int] = None):
        cfg = full.cfg
        self.full, self.cfg, self.device = full, cfg, full.device
        multi = dist.is_initialized() and dist.get_world_size(group) > 1
        self.tp = dist.get_world_size(group) if multi else 1
        self.rank = dist.get_rank(group) if multi else 0
        tp = self.tp
        if cfg.qk_norm:
            raise ValueError("tensor-parallel decode does not cover per-head q/k normalisation")
        if not (full.is_first and full.is_last):
            raise ValueError("tensor-parallel decode needs the whole model on the rank (no pipeline stage)")
        for name, n in (("n_heads", cfg.n_heads), ("n_kv_heads", cfg.n_kv_heads), ("d_ff", cfg.d_ff), ("vocab", cfg.vocab)):
            if n % tp:
                raise ValueError(f"{name}={n} does not split over {tp} tensor-parallel ranks")
        if (cfg.d_ff // tp) % 8 or (cfg.vocab // tp) % 8:
            raise ValueError("the shards of d_ff and vocab must be multiples of 8 elements (16-byte rows)")
        self.n_heads_local = cfg.n_heads // tp
        self.n_kv_local = cfg.n_kv_heads // tp
        self.qw, self.kvw = self.n_heads_local * cfg.head_dim, self.n_kv_local * cfg.head_dim
        self.f_loc, self.v_loc = cfg.d_ff // tp, cfg.vocab // tp
        self.max_batch = int(max_batch)
        d = cfg.d_model
        per_layer = (self.qw + 2 * self.kvw) * d + d * self.qw + 2 * self.f_loc * d + d * self.f_loc
        self.shard = torch.empty(cfg.n_layers * per_layer, dtype=torch.bfloat16, device=self.device)
        self.wqkv: List[torch.Tensor] = []
        self.wo: List[torch.Tensor] = []
        self.wgu: List[torch.Tensor] = []
        self.wdown: List[torch.Tensor] = []
        off = 0
        for _ in range(cfg.n_layers):
            for store, shape in ((self.wqkv, (self.qw + 2 * self.kvw, d)), (self.wo, (d, self.qw)),
                                 (self.wgu, (2 * self.f_loc, d)), (self.wdown, (d, self.f_loc))):
                n = shape[0] * shape[1]
                store.append(self.shard[off:off + n].view(*shape))
                off += n
        B = self.max_batch
        # few rows (rows x ranks <= 256): the all-reduce is bound by latency and runs as one exchange
        ll_rows = min(B, max(8, 256 // tp)) if one_shot_rows is None else min(B, int(one_shot_rows))
        self.comm = TPCommRegion(3 * B * d * 2 + B * cfg.vocab * 2 + TPCommRegion.ll_bytes(tp, ll_rows, d) + 8192, self.device, group,
                                 comm_mode)
        for name in ("part", "x", "h"):
            self.comm.alloc(name, B * d * 2)
        self.comm.alloc("logits", B * cfg.vocab * 2)
        self.comm.enable_one_shot(ll_rows, d)
        self._ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        self._timed = False
        self.refreshes = 0
        self.refresh()

    # ------------------------------------------------------------------ layout switch: replicated -> tensor parallel
    def _copy(self, src: torch.Tensor, dst: torch.Tensor) -> None:
        """Rows of ``src`` (a 2-D slice, rows possibly strided) into the contiguous ``dst``."""
        rows, cols = src.shape
        check(lib().rpeg_copy2d(src.data_ptr(), src.stride(0) * 2, dst.data_ptr(), dst.stride(0) * 2, rows, cols * 2,
                                torch.cuda.current_stream().cuda_stream), "rpeg_copy2d")

    def refresh(self) -> None:
        """Re-slice the whole model's current weights into this rank's shards (call after every optimizer step)."""
        cfg, p, r = self.cfg, self.full.p, self.rank
        self._ev[0].record()
        for i in range(cfg.n_layers):
            wqkv = p[f"l{i}.wqkv"]
            self._copy(wqkv[r * self.qw:(r + 1) * self.qw], self.wqkv[i][: self.qw])
            k0 = cfg.q_width + r * self.kvw
            self._copy(wqkv[k0:k0 + self.kvw], self.wqkv[i][self.qw:self.qw + self.kvw])
            v0 = cfg.q_width + cfg.kv_width + r * self.kvw
            self._copy(wqkv[v0:v0 + self.kvw], self.wqkv[i][self.qw + self.kvw:])
            self._copy(p[f"l{i}.wo"][:, r * self.qw:(r + 1) * self.qw], self.wo[i])
            gu = p[f"l{i}.w_gate_up"]
            self._copy(gu[r * self.f_loc:(r + 1) * self.f_loc], self.wgu[i][: self.f_loc])
            self._copy(gu[cfg.d_ff + r * self.f_loc: cfg.d_ff + (r + 1) * self.f_loc], self.wgu[i][self.f_loc:])
            self._copy(p[f"l{i}.w_down"][:, r * self.f_loc:(r + 1) * self.f_loc], self.wdown[i])
        self._ev[1].record()
        self._timed = True
        self.refreshes += 1

    @property
    def last_reshard_us(self) -> Optional[float]:
        """Device time of the last ``refresh`` in microseconds (synchronises on its end event)."""
        if not self._timed:
            return None
        self._ev[1].synchronize()
        return 1e3 * self._ev[0].elapsed_time(self._ev[1])

    # ------------------------------------------------------------------ what the generator calls
    def kv_columns(self):
        """(first K column, first V column, KV heads) of this rank's heads inside a full-width QKV activation."""
        cfg = self.cfg
        return cfg.q_width + self.rank * self.kvw, cfg.q_width + cfg.kv_width + self.rank * self.kvw, self.n_kv_local

    def forward(self, *args, **kwargs):
        """Prefill runs the whole local model (replicated over the ranks); the generator keeps this rank's K/V heads."""
        return self.full.forward(*args, **kwargs)

    def lm_logits(self, xf: torch.Tensor, decode: bool = False) -> torch.Tensor:
        if not decode:
            return self.full.lm_logits(xf)
        B, V = xf.shape[0], self.cfg.vocab
        logits = self.comm.view("logits", (B, V))
        head = self.full.p["lm_head"][self.rank * self.v_loc:(self.rank + 1) * self.v_loc]
        K.gemm(xf, head, out=logits[:, self.rank * self.v_loc:(self.rank + 1) * self.v_loc])
        self.comm.allgather_cols("logits", B, self.v_loc, V)
        return logits

    @staticmethod
    def _row_parallel(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, ws: torch.Tensor) -> None:
        """This rank's partial sum of a row-parallel linear as ONE bf16 matrix (what the all-reduce reads). A short
        contraction (many ranks) runs as a plain GEMM with 128-column tiles: 2 x 32 CTAs each walk the whole K and no
        second kernel is needed. A long one (few ranks) is cut along K so that every SM streams a slice of the
        weights, and the fp32 partials are summed by the split-K reduction."""
        if a.shape[1] <= 1536:
            K.gemm(a, w, out=out, bn=128, chain=True)
        else:
            K.gemm(a, w, out=out, workspace=ws)

    def decode_step(self, token: torch.Tensor, pos: torch.Tensor, slot_ids: torch.Tensor, seq_len: torch.Tensor,
                    page_table: torch.Tensor, kcache: List[torch.Tensor], vcache: List[torch.Tensor], nsplit: int = 1,
                    groups=None) -> torch.Tensor:
        """One step for ``B`` slots on this rank's shards; returns the final normalised hidden ``[B, d]`` (identical on
        every rank). ``kcache`` / ``vcache`` hold this rank's KV heads only."""
        cfg, p, R = self.cfg, self.full.p, self.comm
        B, d = token.shape[0], cfg.d_model
        if B > self.max_batch:
            raise ValueError(f"batch {B} exceeds the communication buffers ({self.max_batch} rows)")
        ws = self.full._workspace()
        scale = 1.0 / math.sqrt(cfg.head_dim)
        h, x, part = R.view("h", (B, d)), R.view("x", (B, d)), R.view("part", (B, d))
        K.embed_fwd(token, p["embed"], out=h)
        x0, _, _ = K.rmsnorm_fwd(h, p["l0.attn_norm"], cfg.rms_eps)
        qkv = torch.empty((B, self.qw + 2 * self.kvw), dtype=torch.bfloat16, device=self.device)
        xin = x0
        one_shot = R.one_shot(B, d)     # few rows: the all-reduce sums the split-K slabs itself, one kernel fewer per GEMM

        def reduce_into(a, wmat, norm_w, h_out):
            if one_shot:
                R.allreduce_rmsnorm("part", h, norm_w, "x", h_out, B, d, cfg.rms_eps, parts=K.gemm_partials(a, wmat, ws))
            else:
                self._row_parallel(a, wmat, part, ws)
                R.allreduce_rmsnorm("part", h, norm_w, "x", h_out, B, d, cfg.rms_eps)

        for i in range(cfg.n_layers):
            parts = K.gemm_partials(xin, self.wqkv[i], ws)
            K.rope_kv_append_partials_(parts, qkv, 0, self.qw, self.qw + self.kvw, slot_ids, pos, self.full.cos_t, self.full.sin_t,
                                       page_table, kcache[i], vcache[i], self.n_heads_local, self.n_kv_local, cfg.head_dim)
            attn = K.paged_decode_attn(qkv, 0, kcache[i], vcache[i], page_table, seq_len, self.n_heads_local, self.n_kv_local,
                                       cfg.head_dim, scale, nsplit=nsplit, groups=groups)
            reduce_into(attn, self.wo[i], p[f"l{i}.mlp_norm"], "h")
            parts = K.gemm_partials(x, self.wgu[i], ws)
            act = K.swiglu_fwd_partials(parts)
            last = i + 1 == cfg.n_layers
            reduce_into(act, self.wdown[i], p["final_norm"] if last else p[f"l{i + 1}.attn_norm"], None if last else "h")
            xin = x
        return x

    # ------------------------------------------------------------------ start-up check
    def selfcheck(self, rows=(8, 64), steps: int = 2) -> float:
        """Decode ``steps`` tokens for a few rows with this tensor-parallel view and with the whole local model (scratch
        KV caches of one page per row) and return the largest relative difference of the final hidden states over all
        ranks. ``rows`` should cover both all-reduce kernels (rows x ranks <= 256 and above). Raises what a kernel
        reported in the status word (a peer that did not answer). Cheap enough to run once before a long job."""
        cfg, dev = self.cfg, self.device
        worst = 0.0
        for B in rows:
            B = min(int(B), self.max_batch)
            pages = B + 1
            i32 = dict(dtype=torch.int32, device=dev)
            kc_f = [torch.zeros(pages, cfg.n_kv_heads, K.KV_PAGE, cfg.head_dim, dtype=torch.bfloat16, device=dev) for _ in range(cfg.n_layers)]
            vc_f = [torch.zeros_like(t) for t in kc_f]
            kc_t = [torch.zeros(pages, self.n_kv_local, K.KV_PAGE, cfg.head_dim, dtype=torch.bfloat16, device=dev) for _ in range(cfg.n_layers)]
            vc_t = [torch.zeros_like(t) for t in kc_t]
            table = (torch.arange(B, **i32) + 1).view(B, 1).contiguous()
            slot_ids = torch.arange(B, **i32)
            g = torch.Generator(device="cpu").manual_seed(1234 + B)
            for t in range(steps):
                tok = torch.randint(0, cfg.vocab, (B,), generator=g, dtype=torch.int32).to(dev)
                pos = torch.full((B,), t, **i32)
                seq = torch.full((B,), t + 1, **i32)
                want = self.full.decode_step(tok, pos, slot_ids, seq, table, kc_f, vc_f, nsplit=1).float()
                got = self.decode_step(tok, pos, slot_ids, seq, table, kc_t, vc_t, nsplit=1).float()
                worst = max(worst, float(((got - want).abs().max() / want.abs().max().clamp_min(1e-6)).item()))
            del kc_f, vc_f, kc_t, vc_t
        K.check_status()
        if self.tp > 1:
            t = torch.tensor([worst], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            worst = float(t.item())
        return worst

