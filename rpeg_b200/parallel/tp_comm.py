"""Symmetric communication region of the tensor-parallel decode step.

One region per rank, the same layout on every rank: named buffers at fixed byte offsets plus two flag arrays.
Kernels address a buffer as ``peer base + offset`` (any rank's copy) or ``multicast base + offset`` (all copies at
once through NVSwitch: ``multimem.ld_reduce`` adds the ranks' copies in the switch, ``multimem.st`` writes all of
them). The region comes from ``torch.distributed._symmetric_memory`` when it offers a multicast mapping (NVLS);
otherwise, or with ``RPEG_TP_COMM=peer``, from this package's own CUDA-IPC symmetric buffers and the kernels use one
load / store per peer. ``world == 1`` needs no peers at all and runs the same kernels on a private buffer.

The collectives are ``csrc/tp_decode.cu``: ``allreduce_rmsnorm`` (reduce-scatter + residual + RMSNorm + all-gather of
a row-parallel linear's partial sums, one launch) and ``allgather_cols`` (vocabulary-parallel logits). They replace
the NCCL all-reduces and the logits all-gather of the reference's tensor-parallel generation
(RPEG/runtime/workers/megatron_worker.py:2078, 2301-3107).
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import kernels as K
from ..ops._lib import check, lib

WAIT_NS = 5_000_000_000      # ranks replay the same step, but their hosts may be apart by a graph capture or a collection pause
_FLAG_BYTES = 256        # two flag arrays of MAX_PEERS uint32 (column all-gather), then two arrival counters (all-reduce)


def _align(n: int, a: int = 256) -> int:
    return (int(n) + a - 1) // a * a


class TPCommRegion:
    def __init__(self, nbytes: int, device, group=None, mode: Optional[str] = None):
        self.device = torch.device(device)
        self.group = group
        multi = dist.is_initialized() and dist.get_world_size(group) > 1
        self.world = dist.get_world_size(group) if multi else 1
        self.rank = dist.get_rank(group) if multi else 0
        if self.world > K.MAX_PEERS:
            raise ValueError(f"at most {K.MAX_PEERS} ranks in a tensor-parallel group")
        self.nbytes = _align(nbytes + _FLAG_BYTES + 256)
        self.mode = (mode or os.environ.get("RPEG_TP_COMM", "auto")).lower()
        self.mc_ptr = 0
        self._keep = None
        self.backend = "local"
        if self.world == 1:
            self.bytes_view = torch.zeros(self.nbytes, dtype=torch.uint8, device=self.device)
            self.peer_ptrs = [self.bytes_view.data_ptr()]
        else:
            if self.mode in ("auto", "nvls"):
                try:
                    self._open_multicast()
                except Exception as exc:  # noqa: BLE001 - any failure of the optional mapping falls back to peer access
                    self.multicast_error = f"{type(exc).__name__}: {exc}"
                # all ranks use the multicast mapping or none does
                ok = torch.tensor([1 if self._keep is not None else 0], device=self.device)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
                if int(ok.item()) == 0:
                    if self.mode == "nvls":
                        raise RuntimeError("NVLS multicast region requested but not available on every rank: "
                                           + str(getattr(self, "multicast_error", "a peer failed to map it")))
                    self._keep, self.mc_ptr, self.backend = None, 0, "local"
            if self._keep is None:
                from .symm import SymmetricBuffer
                buf = SymmetricBuffer(self.nbytes, self.device, group, zero=True)
                self._keep = buf
                self.bytes_view = buf.bytes_view
                self.peer_ptrs = list(buf.peer_ptrs)
                self.backend = "cuda-ipc peer memory"
        self._cursor = 0
        self.ll_rows, self._ll_d = 0, 0
        self.offsets: Dict[str, Tuple[int, int]] = {}
        self.flag_off = self.nbytes - _align(_FLAG_BYTES)
        self.state = torch.zeros(4, dtype=torch.int32, device=self.device)      # [calls finished, blocks finished, arrivals counted: landed, ready]
        self._peer_array = (ctypes.c_void_p * self.world)(*self.peer_ptrs)
        if self.world > 1:
            torch.cuda.synchronize(self.device)
            dist.barrier(group=group)

    def _open_multicast(self) -> None:
        import torch.distributed._symmetric_memory as symm_mem
        grp = self.group if self.group is not None else dist.group.WORLD
        t = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
        hdl = symm_mem.rendezvous(t, group=grp)
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
        if mc == 0:
            raise RuntimeError("the symmetric allocation has no multicast address on this machine")
        t.zero_()
        self._keep = (t, hdl)
        self.bytes_view = t
        self.peer_ptrs = [int(p) for p in hdl.buffer_ptrs]
        self.mc_ptr = mc
        self.backend = "nvls multicast"

    # ------------------------------------------------------------------ layout
    def alloc(self, name: str, nbytes: int) -> int:
        off = self._cursor
        if off + _align(nbytes) > self.flag_off:
            raise MemoryError(f"communication region of {self.nbytes} bytes is full at '{name}'")
        self._cursor += _align(nbytes)
        self.offsets[name] = (off, int(nbytes))
        return off

    @staticmethod
    def ll_bytes(world: int, rows: int, d: int) -> int:
        """Slot bytes of the one-shot all-reduce: two sets (call parity) x senders x rows x d/2 units of 8 bytes."""
        return 2 * world * rows * d * 4

    def enable_one_shot(self, rows: int, d: int) -> None:
        """Reserve the slots of the one-shot all-reduce: calls of ``allreduce_rmsnorm`` with at most ``rows`` rows of width
        ``d`` then push their partial sums to every rank in self-validating 8-byte units and reduce locally (one
        exchange, for the latency-bound tail of a generation) instead of reduce-scatter + all-gather (three)."""
        if rows <= 0:
            return
        self.alloc("ll", self.ll_bytes(self.world, rows, d))
        self.ll_rows, self._ll_d = int(rows), int(d)

    def view(self, name: str, shape, dtype=torch.bfloat16) -> torch.Tensor:
        off, nbytes = self.offsets[name]
        n = 1
        for s in shape:
            n *= int(s)
        item = torch.empty(0, dtype=dtype).element_size()
        if n * item > nbytes:
            raise ValueError(f"view of '{name}' larger than its {nbytes} bytes")
        return self.bytes_view[off:off + n * item].view(dtype).view(*shape)

    # ------------------------------------------------------------------ collectives
    def one_shot(self, B: int, d: int) -> bool:
        """Whether ``allreduce_rmsnorm`` of ``B`` rows of width ``d`` runs as one exchange (and accepts ``parts``)."""
        return bool(self.ll_rows) and B <= self.ll_rows and d == self._ll_d

    def allreduce_rmsnorm(self, part: str, res: Optional[torch.Tensor], w: torch.Tensor, y: str, h: Optional[str], B: int,
                          d: int, eps: float, parts=None) -> None:
        """``y = rmsnorm(sum over ranks of part + res) * w`` and ``h`` = that sum in bf16, complete in every rank's
        region when the call's kernel has finished. ``parts`` (an ``ops.kernels.Partials`` of a split-K GEMM, only when
        ``one_shot(B, d)``): this rank's partial sum is the sum of those fp32 slabs instead of the ``part`` buffer."""
        if self.one_shot(B, d):
            check(lib().rpeg_tp_allreduce_rmsnorm_ll(self._peer_array, self.mc_ptr or None, self.rank, self.world, self.offsets[part][0],
                                                     None if parts is None else parts.buf.data_ptr(), 0 if parts is None else parts.splits,
                                                     0 if parts is None else parts.stride,
                                                     None if res is None else res.data_ptr(), w.data_ptr(), self.offsets[y][0],
                                                     -1 if h is None else self.offsets[h][0], B, d, eps, self.offsets["ll"][0],
                                                     self.ll_rows, self.state.data_ptr(), WAIT_NS, K.status_word(self.device).data_ptr(),
                                                     torch.cuda.current_stream().cuda_stream), "rpeg_tp_allreduce_rmsnorm_ll")
            return
        if parts is not None:
            raise ValueError("split-K partials are only taken by the one-shot all-reduce")
        check(lib().rpeg_tp_allreduce_rmsnorm(self._peer_array, self.mc_ptr or None, self.rank, self.world, self.offsets[part][0],
                                              None if res is None else res.data_ptr(), w.data_ptr(), self.offsets[y][0],
                                              -1 if h is None else self.offsets[h][0], B, d, eps, self.flag_off,
                                              self.state.data_ptr(), WAIT_NS, K.status_word(self.device).data_ptr(),
                                              torch.cuda.current_stream().cuda_stream), "rpeg_tp_allreduce_rmsnorm")

    @staticmethod
    def trace(enable: bool):
        """Switch the time stamps inside the one-shot all-reduce kernel on or off; returns, for the last traced launch,
        microseconds from its start to (push issued, all senders' units complete)."""
        import ctypes as _ct
        out = (_ct.c_ulonglong * 2)()
        check(lib().rpeg_tp_trace(int(bool(enable)), out), "rpeg_tp_trace")
        return int(out[0]) / 1e3, int(out[1]) / 1e3

    def allgather_cols(self, buf: str, B: int, n_loc: int, ld: int) -> None:
        """Every rank's column block ``[:, rank*n_loc : (rank+1)*n_loc]`` of the ``[B, ld]`` buffer goes to all ranks."""
        if self.world == 1:
            return
        check(lib().rpeg_tp_allgather_cols(self._peer_array, self.mc_ptr or None, self.rank, self.world, self.offsets[buf][0], B,
                                           n_loc, ld, self.flag_off, self.state.data_ptr(), WAIT_NS,
                                           K.status_word(self.device).data_ptr(), torch.cuda.current_stream().cuda_stream),
              "rpeg_tp_allgather_cols")

    def close(self) -> None:
        if self.world > 1:
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
        keep, self._keep = self._keep, None
        self.bytes_view = None
        if hasattr(keep, "close"):
            keep.close()
