"""Versioned hand-over of data between disjoint sets of GPUs through peer memory: weights from the training
ranks to the generation ranks (``WeightChannel``) and rollout rows the other way (``RolloutChannel``).

Both channels keep ``slots`` copies of the payload on the consuming ranks and one version word per (slot,
producer). A producer writes its share straight into the consumer's memory over NVLink (copy kernels on its own
stream) and then release-stores the version number into the consumer's flag word (``publish_version``); a
consumer that finds every producer's word at the version it needs owns a complete copy. Nobody calls NCCL and
nobody synchronises with the host of the other side, so a generation step of iteration ``k + 1`` can run while
the trainers are still in iteration ``k`` (bounded staleness).

Slot arithmetic for staleness ``tau``: iteration ``k`` (1-based) consumes weight version ``max(0, k - 1 - tau)``
and produces version ``k``; the versions that can be live at the same time span ``tau + 2`` numbers, so
``slots = tau + 2`` and version ``v`` lives in slot ``v % slots``. A producer can only be asked for version ``k``
after the rollouts of iteration ``k`` were consumed, which needed version ``k - 1 - tau`` - the previous tenant of
slot ``k % slots`` is ``k - tau - 2`` and no longer read by anyone; the same argument in the other direction
covers the rollout slots. No acknowledgement traffic is needed.

Waiting is split in two: long waits (the other side is still computing, seconds) are host loops around a kernel
that polls for at most ``POLL_S``; the last stretch is folded into the first GEMM that reads the new weights
(``ops.kernels.gemm(..., gate=...)``), whose producer warp checks the same version words before its first TMA
load.

Reference: weight versions and their consumers in RPEG/runtime/weight_versions.py:25-90 and the dataflow table
RPEG/runtime/dataflow.md:74-81; the transfers themselves in RPEG/runtime/semantic_worker.py:6289-6535 (weights)
and :746-970 (rollout artifacts, indexed by global sample id).
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..ops import kernels as K
from ..ops._lib import check, lib
from .symm import SymmetricBuffer

POLL_S = 0.5                 # bound of one device-side poll
MAX_PRODUCERS = 8


def consumed_version(step: int, tau: int) -> int:
    """Weight version that iteration ``step`` (1-based) generates with (RPEG/runtime/weight_versions.py:25)."""
    return max(0, step - 1 - tau)


def slots_for(tau: int) -> int:
    return tau + 2


class _Channel:
    def __init__(self, device, group, producers: Sequence[int], consumers: Sequence[int], slots: int):
        self.device = torch.device(device)
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.producers, self.consumers = list(producers), list(consumers)
        if len(self.producers) > MAX_PRODUCERS:
            raise ValueError(f"at most {MAX_PRODUCERS} producers")
        self.slots = slots
        self.is_producer = self.rank in self.producers
        self.is_consumer = self.rank in self.consumers
        self.flags = SymmetricBuffer(slots * MAX_PRODUCERS * 4, self.device, group, zero=True)
        self._result = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.published_bytes = 0

    def _flag_view(self, slot: int) -> torch.Tensor:
        words = self.flags.tensor(torch.int32)
        return words[slot * MAX_PRODUCERS: slot * MAX_PRODUCERS + len(self.producers)]

    def _signal(self, slot: int, version: int) -> None:
        pi = self.producers.index(self.rank)
        K.publish_version([self.flags.peer_ptrs[c] for c in self.consumers], slot * MAX_PRODUCERS + pi, version)

    def ready(self, version: int, timeout_s: float = 0.0) -> bool:
        """Consumer side: has every producer delivered ``version``? Polls on the device for at most
        ``timeout_s`` in slices of ``POLL_S`` (each slice is one short kernel, so the context stays responsive)."""
        slot = version % self.slots
        deadline = time.monotonic() + timeout_s
        while True:
            K.wait_flags(self._flag_view(slot), version, min(POLL_S, max(1e-4, timeout_s)), self._result)
            if int(self._result.item()) == 1:
                return True
            if time.monotonic() >= deadline:
                return False

    def close(self) -> None:
        self.flags.close()


class WeightChannel(_Channel):
    """``slots`` copies of a flat bf16 parameter vector on every consumer; producer ``i`` of ``P`` pushes the
    ``i``-th contiguous share of the vector to every consumer."""

    def __init__(self, n_params: int, device, group, producers: Sequence[int], consumers: Sequence[int], tau: int = 0):
        super().__init__(device, group, producers, consumers, slots_for(tau))
        self.n = int(n_params)
        self.tau = tau
        # Only consumers hold the copies; the other ranks take part in the exchange of handles with a stub.
        nbytes = self.slots * self._slot_bytes() if self.is_consumer else 256
        self.store = SymmetricBuffer(nbytes, self.device, group)

    def _slot_bytes(self) -> int:
        return (self.n * 2 + 255) // 256 * 256

    def share(self, producer_index: int) -> Tuple[int, int]:
        """Element range ``[lo, hi)`` that producer ``producer_index`` pushes (multiples of 8 elements)."""
        P = len(self.producers)
        per = ((self.n + P - 1) // P + 7) // 8 * 8
        lo = min(self.n, producer_index * per)
        return lo, min(self.n, lo + per)

    def slot_weights(self, version: int) -> torch.Tensor:
        """Consumer side: the bf16 vector of ``version``'s slot (valid once ``ready(version)``)."""
        off = (version % self.slots) * self._slot_bytes()
        return self.store.tensor(torch.bfloat16, self.n, byte_offset=off)

    def seed(self, weights: torch.Tensor) -> None:
        """Consumer side: install version 0 locally (both sides start from the same initial weights)."""
        self.slot_weights(0).copy_(weights[: self.n])

    def publish(self, weights: torch.Tensor, version: int) -> None:
        """Producer side, on the current stream: push this rank's share of ``weights`` into slot
        ``version % slots`` of every consumer, then raise the version words."""
        if not self.is_producer:
            raise RuntimeError("publish() on a rank that is not a producer")
        lo, hi = self.share(self.producers.index(self.rank))
        slot = version % self.slots
        stream = torch.cuda.current_stream().cuda_stream
        nbytes = (hi - lo) * 2
        if nbytes > 0:
            for c in self.consumers:
                dst = self.store.peer_ptrs[c] + slot * self._slot_bytes() + lo * 2
                check(lib().rpeg_copy2d(weights.data_ptr() + lo * 2, nbytes, dst, nbytes, 1, nbytes, stream), "rpeg_copy2d")
                self.published_bytes += nbytes
        self._signal(slot, version)

    def gate(self, version: int, timeout_s: float = 1.0):
        """Argument for ``ops.kernels.gemm(..., gate=...)``: the GEMM reads no tile of the slot before ``version`` is complete."""
        return (self._flag_view(version % self.slots), version, timeout_s)

    def close(self) -> None:
        self.store.close()
        super().close()


class RolloutChannel(_Channel):
    """Rollout rows (response ids, sampling log-probs, lengths) from the generation ranks to the training ranks.

    The global batch of ``n_rows`` rows is cut into equal contiguous blocks, one per consumer; every producer
    scatters the rows it generated by their global index (``scatter_rows_by_index``) and then raises its version
    word with the iteration number."""

    def __init__(self, n_rows: int, max_new: int, device, group, producers: Sequence[int], consumers: Sequence[int], tau: int = 0):
        super().__init__(device, group, producers, consumers, slots_for(tau))
        if n_rows % len(consumers):
            raise ValueError("rows must divide evenly over the consuming ranks")
        self.n_rows, self.T = n_rows, max_new
        self.rows_per_consumer = n_rows // len(consumers)
        self.row_bytes = {"ids": max_new * 4, "logp": max_new * 4, "len": 16}
        self._off: Dict[str, int] = {}
        off = 0
        for name, rb in self.row_bytes.items():
            self._off[name] = off
            off += (self.rows_per_consumer * rb + 255) // 256 * 256
        self._slot_bytes = off
        self.store = SymmetricBuffer(self.slots * off if self.is_consumer else 256, self.device, group, zero=True)

    def _ptrs(self, name: str, slot: int):
        import ctypes
        # the scatter kernel indexes destinations by "owner = global index // rows per consumer"
        return (ctypes.c_void_p * len(self.consumers))(*[self.store.peer_ptrs[c] + slot * self._slot_bytes + self._off[name]
                                                          for c in self.consumers])

    def send(self, step: int, global_idx: torch.Tensor, resp_ids: torch.Tensor, logp: torch.Tensor, lens: torch.Tensor) -> None:
        """Producer side: rows ``global_idx [n]`` (int64) of iteration ``step``."""
        slot = step % self.slots
        lens16 = torch.zeros((lens.numel(), 4), dtype=torch.int32, device=self.device)
        lens16[:, 0] = lens.to(torch.int32)
        nc = len(self.consumers)
        for name, t in (("ids", resp_ids.to(torch.int32).contiguous()), ("logp", logp.float().contiguous()), ("len", lens16)):
            K.scatter_rows_by_index(t, global_idx, self.rows_per_consumer, self._ptrs(name, slot), nc)
            self.published_bytes += t.numel() * t.element_size()
        self._signal(slot, step)

    def receive(self, step: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Consumer side (after ``ready(step)``): this rank's block ``(ids [n, T] int32, logp [n, T] fp32, lens [n] int32)``."""
        base = (step % self.slots) * self._slot_bytes
        n, T = self.rows_per_consumer, self.T
        ids = self.store.tensor(torch.int32, n * T, byte_offset=base + self._off["ids"]).view(n, T)
        logp = self.store.tensor(torch.float32, n * T, byte_offset=base + self._off["logp"]).view(n, T)
        lens = self.store.tensor(torch.int32, n * 4, byte_offset=base + self._off["len"]).view(n, 4)[:, 0]
        return ids, logp, lens

    def close(self) -> None:
        self.store.close()
        super().close()
