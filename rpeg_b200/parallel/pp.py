"""Pipeline parallelism: 1F1B over NCCL point-to-point transfers.

Every rank of a pipeline group holds one stage (``LlamaModel(..., stage=(index, n_stages))``): a contiguous block
of layers, the embedding on the first stage, final norm and heads on the last. A training step runs the
non-interleaved 1F1B order: stage ``s`` of ``p`` does ``min(p - s - 1, m)`` warm-up forwards, then alternates one
forward and one backward, then drains the remaining backwards, so at most ``p - s`` microbatches keep activations
alive. The hidden states ``[T, d]`` (bf16) travel forward, their gradients backward.

Transport is NCCL send/recv (the one transport that stays a library call in this framework; the payload is a
plain contiguous copy and needs no compute fused into it). Each exchange is ONE batched call so that a send and
the receive it is paired with on the neighbour are enqueued together (two ranks that each enqueue a large send
before their receive would wait on each other). The calls run on NCCL's own stream: a send is only waited for
when its buffer is about to be dropped, so it overlaps the next compute; a receive is waited for right before the
kernels that read it.

All stages receive the same packed microbatches (token ids, positions, sequence boundaries: a few KB), so the
shapes of every transfer are known without a handshake.

Reference: Megatron's ``get_forward_backward_func`` 1F1B schedule with ``batch_p2p_comm=True`` as driven by
RPEG/runtime/workers/megatron_worker.py:1657,3808 and :698; results relayed from the last stage to all others with
point-to-point calls in :2035-2077 (``broadcast_from_last`` here).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def one_f_one_b(stage: int, n_stages: int, n_micro: int) -> List[Tuple[str, int]]:
    """The order of forward (``"F"``) and backward (``"B"``) microbatches on ``stage``."""
    if not 0 <= stage < n_stages:
        raise ValueError("stage out of range")
    warm = min(n_stages - stage - 1, n_micro)
    order: List[Tuple[str, int]] = [("F", i) for i in range(warm)]
    f, b = warm, 0
    while f < n_micro:
        order.append(("F", f))
        order.append(("B", b))
        f += 1
        b += 1
    while b < n_micro:
        order.append(("B", b))
        b += 1
    return order


def peak_live_microbatches(stage: int, n_stages: int, n_micro: int) -> int:
    """How many microbatches hold activations at once on ``stage`` under ``one_f_one_b``."""
    live = peak = 0
    for kind, _ in one_f_one_b(stage, n_stages, n_micro):
        live += 1 if kind == "F" else -1
        peak = max(peak, live)
    return peak


class PipelineRunner:
    """Drives one stage through a 1F1B step.

    ``model`` is this rank's stage. ``group`` is the pipeline group (ranks ordered by stage); ``None`` means the
    default group. With ``n_stages == 1`` the runner degenerates to the plain forward/backward loop."""

    def __init__(self, model, group=None):
        self.model = model
        self.group = group
        self.n_stages = dist.get_world_size(group) if dist.is_initialized() else 1
        self.stage = dist.get_rank(group) if dist.is_initialized() else 0
        if model.stage is not None and tuple(model.stage) != (self.stage, self.n_stages):
            raise ValueError(f"model was built for stage {model.stage}, the group says {(self.stage, self.n_stages)}")
        if model.stage is None and self.n_stages > 1:
            raise ValueError("a pipeline group of more than one rank needs stage models")
        self.first, self.last = self.stage == 0, self.stage == self.n_stages - 1
        self._pending: List[Tuple[object, torch.Tensor]] = []   # sends in flight: (work, buffer kept alive)
        if self.n_stages > 1:
            # Build the communicator and both neighbour connections now, all ranks together: NCCL sets a point-to-point
            # connection up on first use with a host-side handshake, which is better done outside the schedule.
            dev = model.device
            dist.all_reduce(torch.zeros(1, device=dev), group=group)
            ops, bufs = [], []
            for peer in (self.stage - 1, self.stage + 1):
                if 0 <= peer < self.n_stages:
                    out, inp = torch.zeros(4, device=dev), torch.zeros(4, device=dev)
                    bufs += [out, inp]
                    ops += [dist.P2POp(dist.isend, out, self._global(peer), group), dist.P2POp(dist.irecv, inp, self._global(peer), group)]
            for w in dist.batch_isend_irecv(ops):
                w.wait()
            torch.cuda.synchronize(dev)
        self.sent_bytes = 0
        self.p2p_calls = 0

    # ------------------------------------------------------------------ transport
    def _global(self, stage: int) -> int:
        return dist.get_global_rank(self.group, stage) if self.group is not None else stage

    def _exchange(self, send: Optional[Tuple[torch.Tensor, int]], recv: Optional[Tuple[torch.Tensor, int]]):
        """One batched call with at most one send and one receive. Returns the receive's work handles."""
        ops = []
        if send is not None:
            ops.append(dist.P2POp(dist.isend, send[0], self._global(send[1]), self.group))
        if recv is not None:
            ops.append(dist.P2POp(dist.irecv, recv[0], self._global(recv[1]), self.group))
        if not ops:
            return []
        works = dist.batch_isend_irecv(ops)
        self.p2p_calls += 1
        if send is not None:
            self.sent_bytes += send[0].numel() * send[0].element_size()
            self._pending.append((works, send[0]))
        return works if recv is not None else []

    @staticmethod
    def _wait(works) -> None:
        for w in works:
            w.wait()

    def _drain_sends(self, keep: int = 0) -> None:
        while len(self._pending) > keep:
            works, _buf = self._pending.pop(0)
            self._wait(works)

    # ------------------------------------------------------------------ one step
    def run(self, microbatches: Sequence, head: Optional[Callable] = None, *, train: bool = True) -> List[torch.Tensor]:
        """``microbatches``: objects with ``tokens, pos, cu_seqlens, max_seqlen`` (``engine.batching.PackedBatch``).
        ``head(mb, xf) -> d_xf`` runs on the LAST stage only: it evaluates the loss on the final hidden states
        and returns their gradient (``train=True``) or anything (``train=False``, forward only; the returned
        values are collected). Returns the list of ``head`` results on the last stage, ``[]`` elsewhere."""
        m, p, s = len(microbatches), self.n_stages, self.stage
        model = self.model
        d = model.cfg.d_model
        dev = model.device
        outs: List[torch.Tensor] = []
        ctxs = {}
        d_heads = {}
        order = one_f_one_b(s, p, m) if train else [("F", i) for i in range(m)]
        n_tok = [int(mb.tokens.numel()) for mb in microbatches]

        def buf(i):
            return torch.empty((n_tok[i], d), dtype=torch.bfloat16, device=dev)

        # Receives are posted one operation ahead: while operation k computes, the input of operation k + 1 is
        # already on its way. next_in[k] = (kind, microbatch, buffer, works).
        def post_recv(k, send=None):
            if k >= len(order):
                self._exchange(send, None)
                return None
            kind, i = order[k]
            if kind == "F" and not self.first:
                b = buf(i)
                return (b, self._exchange(send, (b, s - 1)))
            if kind == "B" and not self.last:
                b = buf(i)
                return (b, self._exchange(send, (b, s + 1)))
            self._exchange(send, None)
            return None

        incoming = post_recv(0)
        for k, (kind, i) in enumerate(order):
            mb = microbatches[i]
            if incoming is not None:
                x_in, works = incoming
                self._wait(works)
            else:
                x_in = None
            if kind == "F":
                y, ctx = model.forward(mb.tokens, mb.pos, mb.cu_seqlens, mb.max_seqlen, keep=train, h_in=x_in)
                if train:
                    ctxs[i] = ctx
                if self.last:
                    if head is not None:
                        r = head(mb, y)
                        if train:
                            d_heads[i] = r
                        else:
                            outs.append(r)
                    incoming = post_recv(k + 1)
                else:
                    incoming = post_recv(k + 1, send=(y, s + 1))
            else:
                d_out = d_heads.pop(i) if self.last else x_in
                d_in = model.backward(ctxs.pop(i), d_out)
                if self.first:
                    incoming = post_recv(k + 1)
                else:
                    incoming = post_recv(k + 1, send=(d_in, s - 1))
            self._drain_sends(keep=2)
        self._drain_sends()
        return outs

    # ------------------------------------------------------------------ results
    def broadcast_from_last(self, t: torch.Tensor) -> torch.Tensor:
        """Make the last stage's tensor (metrics, log-probs) available on every stage (in place)."""
        if self.n_stages > 1:
            dist.broadcast(t, self._global(self.n_stages - 1), group=self.group)
        return t
