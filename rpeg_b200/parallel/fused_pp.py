"""Executor of the fused bidirectional actor/critic pipeline: two pipeline-parallel models share the same GPUs,
the actor with its stages in device order and the critic in reverse order, and every device follows ONE
precomputed instruction stream that interleaves the two models' forward and backward microtasks
(``runtime.fused_pipeline.build_fused_pipeline_schedule``), so one model's work fills the other's bubbles.

One process per GPU. Rank ``r`` holds stage ``r`` of a forward-ordered model and stage ``p - 1 - r`` of a
reverse-ordered one (``LlamaModel(..., stage=...)``) and walks ``schedule.device_order[r]``:

    F task   input from the previous logical stage (NCCL receive) or the token ids (stage 0); forward of the stage;
             output to the next logical stage (NCCL send), or the model's loss head on its last stage
    B task   gradient from the next logical stage (or from the loss head); backward of the stage;
             gradient of the input to the previous logical stage

Transport: every (model, phase) pair has its own NCCL communicator, so its messages form one single-direction,
in-order stream per neighbour pair (the schedule runs each model's forwards, and each model's backwards, in
microbatch order on every stage) and streams of different pairs cannot block each other; sends are asynchronous,
the receive of the next task is posted before the current task computes. The schedule itself is validated
against a blocking-rendezvous simulation when it is built, which is stricter than what this executor needs.

Reference: two colocated worker processes replaying a shared microtask schedule, ordered across processes by CUDA
IPC events or filesystem markers (RPEG/runtime/fused_pipeline.py:287-625, RPEG/runtime/workers/
megatron_worker.py:3376-3806). Here both models live in one process per GPU, so the order is plain stream order.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Sequence, Tuple

import torch
import torch.distributed as dist

from ..runtime.fused_pipeline import FusedPipelineModel, FusedPipelineSchedule, build_fused_pipeline_schedule


def uniform_schedule(n_stages: int, microbatches: Dict[str, int], *, forward_s: float = 1.0, backward_s: float = 2.0,
                     activation_bytes: int = 1, reverse: Sequence[str] = ("critic",)) -> FusedPipelineSchedule:
    """A schedule for models with equal stage costs (what a caller without measured per-stage times uses)."""
    models = [FusedPipelineModel.uniform(name, pipeline_stages=n_stages, microbatches=m, forward_s=forward_s, backward_s=backward_s,
                                         activation_bytes=activation_bytes, reverse=name in reverse)
              for name, m in sorted(microbatches.items())]
    return build_fused_pipeline_schedule(models)


def logical_stage(model: FusedPipelineModel, device: int) -> int:
    """The logical stage of ``model`` that lives on physical stage ``device``."""
    return model.pipeline_stages - 1 - device if model.reverse else device


class FusedPipelineExecutor:
    def __init__(self, stage_models: Dict[str, object], schedule: FusedPipelineSchedule):
        """``stage_models[name]``: this rank's stage of pipeline ``name`` (built with ``stage=(logical_stage(...), p)``).
        Collective: every rank of the default group constructs the executor (it creates the communicators)."""
        self.schedule = schedule
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.spec = {m.name: m for m in schedule.models}
        self.models = stage_models
        for name, m in self.spec.items():
            if m.pipeline_stages != self.world:
                raise ValueError(f"{name}: {m.pipeline_stages} stages on {self.world} ranks")
            want = (logical_stage(m, self.rank), self.world)
            if tuple(stage_models[name].stage) != want:
                raise ValueError(f"{name}: this rank needs stage {want}, the model was built for {stage_models[name].stage}")
        self.comm = {}
        for name in sorted(self.spec):                      # same creation order on every rank
            for phase in ("F", "B"):
                self.comm[(name, phase)] = dist.new_group(list(range(self.world)))
        dev = next(iter(stage_models.values())).device
        # Build every communicator and every neighbour connection now, in the same order on all ranks. NCCL sets a
        # point-to-point connection up on first use with a host-side handshake between the two ranks; left to the
        # instruction streams, rank 0 could sit in the handshake of one communicator while rank 1 sits in another's.
        for key in sorted(self.comm):
            g = self.comm[key]
            dist.all_reduce(torch.zeros(1, device=dev), group=g)
            ops, bufs = [], []
            for peer in (self.rank - 1, self.rank + 1):
                if 0 <= peer < self.world:
                    out, inp = torch.zeros(4, device=dev), torch.zeros(4, device=dev)
                    bufs += [out, inp]
                    ops += [dist.P2POp(dist.isend, out, peer, g), dist.P2POp(dist.irecv, inp, peer, g)]
            if ops:
                for w in dist.batch_isend_irecv(ops):
                    w.wait()
        torch.cuda.synchronize(dev)
        self.tasks = {t.task_id: t for t in schedule.tasks}
        self.order: Tuple[str, ...] = tuple(schedule.device_order[self.rank])
        self.p2p_calls = 0

    # ------------------------------------------------------------------ helpers
    def _needs_recv(self, t) -> bool:
        last = self.spec[t.model].pipeline_stages - 1
        return (t.phase == "F" and t.stage > 0) or (t.phase == "B" and t.stage < last)

    def _peer(self, t, receiving: bool) -> int:
        """Physical stage (= rank) on the other end of ``t``'s input (``receiving``) or output."""
        m = self.spec[t.model]
        if t.phase == "F":
            other = t.stage - 1 if receiving else t.stage + 1
        else:
            other = t.stage + 1 if receiving else t.stage - 1
        return m.device_stage(other)

    def run(self, microbatches: Dict[str, Sequence], heads: Dict[str, Callable]) -> None:
        """``microbatches[name][i]``: packed microbatch ``i`` of pipeline ``name`` (the same on every rank);
        ``heads[name](mb, xf) -> d_xf`` runs on the device that holds ``name``'s last logical stage."""
        pending: Dict[str, Tuple[torch.Tensor, object]] = {}
        sends: List[Tuple[object, torch.Tensor]] = []
        ctxs, d_heads = {}, {}

        def post(i: int) -> None:
            if i >= len(self.order):
                return
            tid = self.order[i]
            t = self.tasks[tid]
            if tid in pending or not self._needs_recv(t):
                return
            model = self.models[t.model]
            n_tok = int(microbatches[t.model][t.microbatch].tokens.numel())
            buf = torch.empty((n_tok, model.cfg.d_model), dtype=torch.bfloat16, device=model.device)
            g = self.comm[(t.model, t.phase)]
            pending[tid] = (buf, dist.batch_isend_irecv([dist.P2POp(dist.irecv, buf, self._peer(t, True), g)]))
            self.p2p_calls += 1

        def send(t, tensor: torch.Tensor) -> None:
            g = self.comm[(t.model, t.phase)]
            sends.append((dist.batch_isend_irecv([dist.P2POp(dist.isend, tensor, self._peer(t, False), g)]), tensor))
            self.p2p_calls += 1
            while len(sends) > 4:                            # keep a few in flight, release the older buffers
                ws, _ = sends.pop(0)
                for w in ws:
                    w.wait()

        post(0)
        for i, tid in enumerate(self.order):
            post(i + 1)
            t = self.tasks[tid]
            model = self.models[t.model]
            mb = microbatches[t.model][t.microbatch]
            last = self.spec[t.model].pipeline_stages - 1
            x_in = None
            if tid in pending:
                x_in, works = pending.pop(tid)
                for w in works:
                    w.wait()
            key = (t.model, t.microbatch)
            if t.phase == "F":
                y, ctx = model.forward(mb.tokens, mb.pos, mb.cu_seqlens, mb.max_seqlen, keep=True, h_in=x_in)
                ctxs[key] = ctx
                if t.stage == last:
                    d_heads[key] = heads[t.model](mb, y)
                else:
                    send(t, y)
            else:
                d_out = d_heads.pop(key) if t.stage == last else x_in
                d_in = model.backward(ctxs.pop(key), d_out)
                if t.stage > 0:
                    send(t, d_in)
        for ws, _ in sends:
            for w in ws:
                w.wait()

    def broadcast_from_last(self, name: str, t: torch.Tensor) -> torch.Tensor:
        """Make the tensor of the rank that holds ``name``'s last logical stage available everywhere (in place)."""
        m = self.spec[name]
        dist.broadcast(t, m.device_stage(m.pipeline_stages - 1))
        return t
