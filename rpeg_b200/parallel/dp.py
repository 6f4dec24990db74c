"""Data-parallel context: symmetric weight / gradient buffers and the fused optimizer step.

One process per GPU. Every rank holds the full bf16 weights and full fp32 gradients of a model in
symmetric memory; Adam state exists only for the rank's contiguous shard of the flat parameter
space. ``fused_adam_step`` runs, on each rank's own stream,

    barrier(grads ready) -> dp_reduce_norm -> barrier(+partial norms) -> dp_adam_push -> barrier

where ``dp_reduce_norm`` pulls the owner's shard of every peer's gradient over NVLink and
``dp_adam_push`` stores the updated bf16 shard into every peer's weight buffer: gradient
reduce-scatter, optimizer and parameter all-gather without an NCCL call or a host sync. The
barriers are device-side flag exchanges with a bounded wait (a timeout surfaces through
``ops.kernels.check_status``).

Reference behaviour being replaced: ZeRO-1/2 with NCCL ``reduce_scatter_tensor`` buckets and
``all_gather_into_tensor`` (RPEG/runtime/workers/megatron_worker.py:909-1100, 1246-1285).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import kernels as K
from ..ops._lib import check, lib
from .symm import SignalPad, SymmetricBuffer

BARRIER_TIMEOUT_NS = 60_000_000_000  # ranks may arrive many seconds apart (uneven generation lengths, first-step graph capture)


class DPContext:
    def __init__(self, device, group=None, tag: str = "actor", pad: Optional[SignalPad] = None, slot_base: int = 0):
        self.device = torch.device(device)
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > K.MAX_PEERS:
            raise ValueError(f"at most {K.MAX_PEERS} peers per node")
        self.tag = tag
        self.pad = pad if pad is not None else (SignalPad(self.device, group) if self.world > 1 else None)
        self.slot_base = slot_base
        self.buffers: Dict[str, SymmetricBuffer] = {}
        self._scalar = torch.zeros(1, dtype=torch.float64, device=self.device)
        self._side: Optional[torch.cuda.Stream] = None          # stream of the bucketed gradient reduction
        self._covered: list = []                                # flat ranges reduced under the backward pass of this step
        self._overlap_scale = 1.0

    def clone(self, tag: str) -> "DPContext":
        """Context for another model sharing this one's signal pad (own barrier slots) and buffer table: buffers are
        keyed by tag (``alloc_weights(cfg, tag=...)`` on either context), so the clone finds what was allocated for it."""
        c = DPContext(self.device, self.group, tag, self.pad, self.slot_base + 8)
        c.buffers = self.buffers
        return c

    # -- layout
    def shard_range(self, total: int) -> Tuple[int, int]:
        per = (total + self.world - 1) // self.world
        per = (per + 63) // 64 * 64
        off = min(total, self.rank * per)
        return off, max(0, min(total, off + per) - off)

    def alloc_weights(self, cfg, tag: Optional[str] = None) -> torch.Tensor:
        from ..models.llama import ParamLayout
        n = ParamLayout(cfg).total
        buf = SymmetricBuffer(n * 2, self.device, self.group)
        self.buffers[f"{tag or self.tag}.w"] = buf
        return buf.tensor(torch.bfloat16, n)

    def alloc_grads(self, cfg, tag: Optional[str] = None, extra_bytes: int = 0) -> torch.Tensor:
        from ..models.llama import ParamLayout
        n = ParamLayout(cfg).total
        buf = SymmetricBuffer(max(n * 4, extra_bytes), self.device, self.group, zero=True)
        self.buffers[f"{tag or self.tag}.g"] = buf
        return buf.tensor(torch.float32, n)

    # -- collectives
    def all_reduce_scalar(self, value: float) -> float:
        if self.world == 1:
            return value
        self._scalar.fill_(value)
        dist.all_reduce(self._scalar, group=self.group)
        return float(self._scalar.item())

    def barrier(self, slot: int, payload_in: Optional[torch.Tensor] = None, payload_out: Optional[torch.Tensor] = None) -> None:
        """Device-side barrier on the current stream (no host sync)."""
        if self.world == 1:
            return
        s = self.slot_base + slot
        self.pad.epochs[s] += 1
        check(lib().rpeg_flag_barrier(self.pad.ptr_array(), self.rank, self.world, s, self.pad.epochs[s],
                                      None if payload_in is None else payload_in.data_ptr(),
                                      None if payload_out is None else payload_out.data_ptr(), BARRIER_TIMEOUT_NS,
                                      K.status_word(self.device).data_ptr(), torch.cuda.current_stream().cuda_stream),
              "rpeg_flag_barrier")

    # -- gradient reduction in buckets under the backward pass (ZeRO-2 style overlap)
    def _reduce_range(self, opt, lo: int, hi: int, scale: float) -> None:
        """This rank's part of the flat range ``[lo, hi)``: sum the peers' gradients into ``opt.reduced`` and add the
        squared norm to ``opt.sumsq``, on the current stream."""
        a, b = max(lo, opt.shard_off), min(hi, opt.shard_off + opt.shard_n)
        if a >= b:
            return
        g_buf = self.buffers[f"{self.tag}.g"]
        check(lib().rpeg_dp_reduce_norm(g_buf.ptr_array(), self.world, a, b - a, scale,
                                        opt.reduced.data_ptr() + 4 * (a - opt.shard_off), opt.sumsq.data_ptr(),
                                        torch.cuda.current_stream().cuda_stream), "rpeg_dp_reduce_norm")

    def overlap_hook(self, opt, model, bucket_layers: int = 4, grad_scale: float = 1.0):
        """Hook for ``LlamaModel.grad_hook`` during the LAST microbatch's backward pass of a step: whenever
        ``bucket_layers`` more layers have their final gradients, a side stream waits for that point of the backward,
        meets the peers in a flag barrier (their gradients of the bucket are final too) and reduces this rank's part of
        the bucket, while the main stream goes on with the earlier layers. ``fused_adam_step`` then only reduces what no
        bucket covered (the embedding), waits for the side stream and runs Adam. Reference: backward hooks filling
        buckets for asynchronous ``reduce_scatter_tensor`` calls, at most two in flight
        (RPEG/runtime/workers/megatron_worker.py:909-1100)."""
        if self.world == 1:
            return None
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.device)
        lay = model.layout
        self._covered = []
        self._overlap_scale = float(grad_scale)
        opt.sumsq.zero_()
        lo_l, hi_l = model.layer_lo, model.layer_hi
        tail = lay.entries["final_norm"][0] if "final_norm" in lay.entries else lay.total

        def start_of(layer: int) -> int:
            return lay.entries[f"l{layer}.attn_norm"][0] if layer < hi_l else tail

        def hook(i: int) -> None:
            if (i - lo_l) % bucket_layers != 0:
                return
            lo = start_of(i)
            j = min(i + bucket_layers, hi_l)
            hi = lay.total if j == hi_l else start_of(j)         # the first bucket takes the final norm and the heads along
            ev = torch.cuda.Event()
            ev.record()
            self._side.wait_event(ev)
            with torch.cuda.stream(self._side):
                self.barrier(3)
                self._reduce_range(opt, lo, hi, self._overlap_scale)
            self._covered.append((lo, hi))

        return hook

    def fused_adam_step(self, opt, grad_scale: float = 1.0, after_wait=None) -> None:
        """``after_wait()`` is called once the first barrier is queued: what precedes it on the stream is the wait for
        the slowest rank's backward, what follows is the step itself (callers time the two apart)."""
        w_buf = self.buffers[f"{self.tag}.w"]
        g_buf = self.buffers[f"{self.tag}.g"]
        stream = torch.cuda.current_stream().cuda_stream
        b1, b2 = opt.betas
        self.barrier(0)                                              # every rank finished its backward
        if after_wait is not None:
            after_wait()
        if self._covered:
            # buckets were reduced under the backward pass: what is left of the shard, then join the side stream
            covered, self._covered = sorted(self._covered), []
            at = 0
            total = opt.model.layout.total
            for lo, hi in covered + [(total, total)]:
                if lo > at:
                    self._reduce_range(opt, at, lo, grad_scale)
                at = max(at, hi)
            ev = torch.cuda.Event()
            ev.record(self._side)
            torch.cuda.current_stream().wait_event(ev)
        else:
            opt.sumsq.zero_()
            check(lib().rpeg_dp_reduce_norm(g_buf.ptr_array(), self.world, opt.shard_off, opt.shard_n, grad_scale,
                                            opt.reduced.data_ptr(), opt.sumsq.data_ptr(), stream), "rpeg_dp_reduce_norm")
        self.barrier(1, payload_in=opt.sumsq, payload_out=opt.partials)  # exchange partial squared norms
        check(lib().rpeg_dp_adam_push(opt.master.data_ptr(), opt.m.data_ptr(), opt.v.data_ptr(), opt.reduced.data_ptr(),
                                      w_buf.ptr_array(), self.world, opt.shard_off, opt.shard_n, opt.lr, b1, b2,
                                      opt.eps, opt.wd, opt.step_count, opt.partials.data_ptr(), self.world,
                                      opt.max_grad_norm, stream), "rpeg_dp_adam_push")
        self.barrier(2)                                              # every shard landed everywhere

    def broadcast_weights(self, w: torch.Tensor, src: int = 0) -> None:
        if self.world > 1:
            dist.broadcast(w, src=src, group=self.group)
