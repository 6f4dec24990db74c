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
from .symm import SymmetricBuffer

ROW_BLOCK = 128


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
        self.stage = SymmetricBuffer(max_rows * self.N * 2, self.device, group)                 # [world][M/world][N] bf16
        self.counters = SymmetricBuffer(max(256, max_rows // ROW_BLOCK * 4), self.device, group, zero=True)
        out_rows = max_rows if all_reduce else max_rows // self.world
        self.out = SymmetricBuffer(out_rows * self.N * 2, self.device, group)
        self.epoch = 0
        self._last_m: Optional[int] = None

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        """``x_shard [M, K/p]`` bf16 -> ``[M/world, N]`` (reduce-scatter) or ``[M, N]`` (all-reduce), a view
        of this layer's symmetric output buffer (valid until the next call)."""
        M, Kp = x_shard.shape
        if M % (ROW_BLOCK * self.world) or M > self.max_rows:
            raise ValueError(f"M={M} must be a multiple of {ROW_BLOCK * self.world} and at most {self.max_rows}")
        if self._last_m is not None and self._last_m != M:
            # arrival counters are per 128-row block and count calls: a new M changes which blocks exist
            torch.cuda.synchronize(self.device)
            if self.world > 1:
                dist.barrier(group=self.group)
            self.counters.bytes_view.zero_()
            torch.cuda.synchronize(self.device)
            if self.world > 1:
                dist.barrier(group=self.group)
            self.epoch = 0
        self._last_m = M
        self.epoch += 1
        check(lib().rpeg_gemm_rs(x_shard.data_ptr(), self.w.data_ptr(), M, self.N, Kp, x_shard.stride(0), self.w.stride(0),
                                 self.stage.ptr_array(), self.counters.ptr_array(), self.out.ptr_array(), self.N, self.rank,
                                 self.world, self.epoch, int(self.all_reduce), K.status_word(self.device).data_ptr(),
                                 torch.cuda.current_stream().cuda_stream), "rpeg_gemm_rs")
        rows = M if self.all_reduce else M // self.world
        return self.out.tensor(torch.bfloat16, rows * self.N).view(rows, self.N)

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
        for b in (self.stage, self.counters, self.out):
            b.close()
