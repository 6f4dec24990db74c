"""Tensor-parallel linear layers whose collective is fused into the GEMM kernel.

``RowParallelLinear`` is the second half of a tensor-parallel MLP or attention block: every rank
holds a slice of the contraction dimension (``x_r [M, K/p]``, ``w_r [N, K/p]``), and the sum of the
partial products is needed either scattered by rows (sequence-parallel layout) or on every rank.
``forward`` launches ONE kernel per rank (``csrc/gemm_rs.cu``): tcgen05 tiles whose epilogue pushes the
partial tile over NVLink into the owner's staging buffer, and a tail phase in which each rank sums the
partials of its rows (and, for the all-reduce form, stores the result into every peer's output).
Staging, arrival counters and outputs live in symmetric memory allocated once for the largest shape.

The unfused composition (library GEMM, then NCCL reduce-scatter or all-reduce) is kept as
``forward_unfused`` for tests and for the benchmark that compares the two. Reference: Megatron's
RowParallelLinear under the reference's tensor-parallel groups
(RPEG/runtime/workers/megatron_worker.py:124-303, 676-715).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import kernels as K
from ..ops._lib import check, lib
from .symm import SignalPad, SymmetricBuffer

ROW_BLOCK = 128
BARRIER_TIMEOUT_NS = 30_000_000_000


class RowParallelLinear:
    def __init__(self, weight_shard: torch.Tensor, max_rows: int, device, group=None, all_reduce: bool = False):
        """``weight_shard [N, K/p]`` bf16 (this rank's slice of the input features); ``max_rows`` is the
        largest M (a multiple of ``128 * world``) a call may use."""
        self.w = weight_shard
        self.device = torch.device(device)
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.all_reduce = all_reduce
        self.N = int(weight_shard.shape[0])
        if max_rows % (ROW_BLOCK * self.world):
            raise ValueError(f"max_rows must be a multiple of {ROW_BLOCK * self.world}")
        self.max_rows = max_rows
        # Two sets of staging / counters / output, used alternately: a fast rank may already push the partials of
        # call e+1 while a slow owner still reduces call e, and call e+2 cannot start anywhere before every
        # owner has received (hence finished reducing) call e+1's predecessor.
        out_rows = max_rows if all_reduce else max_rows // self.world
        self.stage = [SymmetricBuffer(max_rows * self.N * 2, self.device, group) for _ in range(2)]   # [world][M/world][N] bf16
        self.counters = [SymmetricBuffer(max(256, max_rows // ROW_BLOCK * 4), self.device, group, zero=True) for _ in range(2)]
        self.out = [SymmetricBuffer(out_rows * self.N * 2, self.device, group) for _ in range(2)]
        # All-reduce mode: an owner stores its reduced rows into every peer's output, and a rank's kernel ends when ITS
        # rows are done, not when the peers' rows have landed here. A flag barrier after the kernel (every rank signals
        # once its own stores are issued and complete) closes that window before the next kernel reads the output.
        self.pad = SignalPad(self.device, group) if (all_reduce and self.world > 1) else None
        self.epoch = 0
        self._last_m: Optional[int] = None

    def use_weight(self, weight_shard: torch.Tensor) -> "RowParallelLinear":
        """Switch to another weight with the same number of output features: layers that run one after the other
        can share one set of staging / counter / output buffers."""
        if int(weight_shard.shape[0]) != self.N:
            raise ValueError(f"shared buffers are sized for {self.N} output features, got {weight_shard.shape[0]}")
        self.w = weight_shard
        return self

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        """``x_shard [M, K/p]`` bf16 -> ``[M/world, N]`` (reduce-scatter) or ``[M, N]`` (all-reduce), a view
        of one of this layer's two symmetric output buffers (valid until the call after the next one)."""
        M, Kp = x_shard.shape
        if M % (ROW_BLOCK * self.world) or M > self.max_rows:
            raise ValueError(f"M={M} must be a multiple of {ROW_BLOCK * self.world} and at most {self.max_rows}")
        if self._last_m is not None and self._last_m != M:
            # arrival counters are per 128-row block and count calls: a new M changes which blocks exist
            torch.cuda.synchronize(self.device)
            if self.world > 1:
                dist.barrier(group=self.group)
            for c in self.counters:
                c.bytes_view.zero_()
            torch.cuda.synchronize(self.device)
            if self.world > 1:
                dist.barrier(group=self.group)
            self.epoch = 0
        self._last_m = M
        self.epoch += 1
        b = self.epoch % 2
        calls = (self.epoch + 1) // 2            # how often this buffer set (and its counters) has been used
        check(lib().rpeg_gemm_rs(x_shard.data_ptr(), self.w.data_ptr(), M, self.N, Kp, x_shard.stride(0), self.w.stride(0),
                                 self.stage[b].ptr_array(), self.counters[b].ptr_array(), self.out[b].ptr_array(), self.N, self.rank,
                                 self.world, calls, int(self.all_reduce), K.status_word(self.device).data_ptr(),
                                 torch.cuda.current_stream().cuda_stream), "rpeg_gemm_rs")
        if self.pad is not None:
            self.pad.epochs[0] += 1
            check(lib().rpeg_flag_barrier(self.pad.ptr_array(), self.rank, self.world, 0, self.pad.epochs[0], None, None,
                                          BARRIER_TIMEOUT_NS, K.status_word(self.device).data_ptr(),
                                          torch.cuda.current_stream().cuda_stream), "rpeg_flag_barrier")
        rows = M if self.all_reduce else M // self.world
        return self.out[b].tensor(torch.bfloat16, rows * self.N).view(rows, self.N)

    def forward_unfused(self, x_shard: torch.Tensor) -> torch.Tensor:
        """Same result from a plain GEMM followed by an NCCL collective (the baseline)."""
        part = K.gemm(x_shard, self.w)
        if self.world == 1:
            return part
        if self.all_reduce:
            dist.all_reduce(part, group=self.group)
            return part
        out = torch.empty((part.shape[0] // self.world, self.N), dtype=part.dtype, device=part.device)
        dist.reduce_scatter_tensor(out, part, group=self.group)
        return out

    def close(self) -> None:
        for b in (*self.stage, *self.counters, *self.out):
            b.close()
        if self.pad is not None:
            self.pad.close()


class ColumnParallelLinear:
    """First half of a tensor-parallel block with a sequence-parallel input: every rank holds ``M / world``
    rows of the activation and a slice ``w_r [N / world, K]`` of the output features. ``forward`` runs a
    device-side barrier (nobody still reads the buffer about to be overwritten) and then ONE kernel
    (``csrc/ag_gemm.cu``) whose copy warps push this rank's rows over NVLink into every peer's copy of ``X`` while
    its tensor-core tiles already work on the rows that are there. ``X`` is double buffered so a rank may write its next input while a slower peer
    still reads the previous one."""

    def __init__(self, weight_shard: torch.Tensor, max_rows: int, device, group=None):
        self.w = weight_shard
        self.device = torch.device(device)
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.N, self.K = int(weight_shard.shape[0]), int(weight_shard.shape[1])
        if max_rows % (ROW_BLOCK * self.world):
            raise ValueError(f"max_rows must be a multiple of {ROW_BLOCK * self.world}")
        self.max_rows = max_rows
        self.x = [SymmetricBuffer(max_rows * self.K * 2, self.device, group) for _ in range(2)]
        self.ready = SymmetricBuffer(2 * (max_rows // ROW_BLOCK) * 4, self.device, group, zero=True)   # arrival counters, one half per X buffer
        self.pad = SignalPad(self.device, group) if self.world > 1 else None
        self.epoch = 0
        self._last_m: Optional[int] = None

    def use_weight(self, weight_shard: torch.Tensor) -> "ColumnParallelLinear":
        """Switch to another weight with the same number of input features (shared input buffers)."""
        if int(weight_shard.shape[1]) != self.K:
            raise ValueError(f"shared buffers are sized for {self.K} input features, got {weight_shard.shape[1]}")
        self.w, self.N = weight_shard, int(weight_shard.shape[0])
        return self

    def input_rows(self, M: int) -> torch.Tensor:
        """This rank's slice ``[M / world, K]`` of the buffer the NEXT ``forward`` call will read: write the
        activation shard here (it is the GEMM's operand, no staging copy)."""
        buf = self.x[(self.epoch + 1) % 2]
        per = M // self.world
        return buf.tensor(torch.bfloat16, M * self.K).view(M, self.K)[self.rank * per:(self.rank + 1) * per]

    def forward(self, M: int) -> torch.Tensor:
        """Consume the shards written through ``input_rows(M)`` on every rank; returns ``y_r [M, N / world]``."""
        if M % (ROW_BLOCK * self.world) or M > self.max_rows:
            raise ValueError(f"M={M} must be a multiple of {ROW_BLOCK * self.world} and at most {self.max_rows}")
        if self._last_m is not None and self._last_m != M:
            torch.cuda.synchronize(self.device)
            if self.world > 1:
                dist.barrier(group=self.group)
            self.ready.bytes_view.zero_()
            self.epoch = self.epoch % 2          # keep the buffer parity, restart the counters
            torch.cuda.synchronize(self.device)
        self._last_m = M
        self.epoch += 1
        buf = self.x[self.epoch % 2]
        stream = torch.cuda.current_stream().cuda_stream
        if self.world > 1:
            self.pad.epochs[0] += 1
            check(lib().rpeg_flag_barrier(self.pad.ptr_array(), self.rank, self.world, 0, self.pad.epochs[0], None, None,
                                          BARRIER_TIMEOUT_NS, K.status_word(self.device).data_ptr(), stream), "rpeg_flag_barrier")
        y = torch.empty((M, self.N), dtype=torch.bfloat16, device=self.device)
        ready = self.ready.ptr_array((self.epoch % 2) * (self.max_rows // ROW_BLOCK) * 4)
        calls = (self.epoch + 1) // 2            # how many times this buffer (and its counters) has been used
        check(lib().rpeg_ag_gemm(buf.ptr_array(), self.w.data_ptr(), y.data_ptr(), ready, M, self.N, self.K, self.K,
                                 self.w.stride(0), self.N, self.rank, self.world, calls, K.status_word(self.device).data_ptr(), stream),
              "rpeg_ag_gemm")
        return y

    def gathered(self, M: int) -> torch.Tensor:
        """All ranks' rows ``[M, K]`` as the last ``forward(M)`` left them in this rank's operand buffer (a view that
        stays valid until the next-but-one ``forward``): weight-gradient GEMMs read the gathered operand from here."""
        return self.x[self.epoch % 2].tensor(torch.bfloat16, M * self.K).view(M, self.K)

    def forward_unfused(self, x_shard: torch.Tensor) -> torch.Tensor:
        """NCCL all-gather followed by a plain GEMM (the baseline)."""
        if self.world == 1:
            return K.gemm(x_shard, self.w)
        full = torch.empty((x_shard.shape[0] * self.world, self.K), dtype=x_shard.dtype, device=x_shard.device)
        dist.all_gather_into_tensor(full, x_shard.contiguous(), group=self.group)
        return K.gemm(full, self.w)

    def close(self) -> None:
        for b in (*self.x, self.ready):
            b.close()
        if self.pad is not None:
            self.pad.close()
