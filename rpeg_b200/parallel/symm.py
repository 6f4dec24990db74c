"""Symmetric buffers across the ranks of one node: same size on every rank, every rank holds a
device pointer to every peer's copy (CUDA IPC over NVLink peer access).

``SymmetricBuffer`` is allocated collectively; ``local`` is a normal torch tensor over this rank's
memory and ``peer_ptrs`` are raw device addresses (this rank's own included, in rank order) that the
fused kernels take. ``SignalPad`` is a small zero-initialised symmetric buffer with flag slots and
a float payload area used by the device-side barrier.

Handles travel over ``torch.distributed`` object collectives (NCCL/Gloo group of the job), so this
layer needs no MPI, UCX or filesystem rendezvous. The reference moves such tensors between
processes through pickled CUDA-IPC storages and ad-hoc NCCL groups
(RPEG/runtime/semantic_worker.py:9840-10028, 11281-11365).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops._lib import check, lib

_DTYPE_STR = {torch.bfloat16: None, torch.float32: "<f4", torch.int32: "<i4", torch.uint8: "|u1", torch.int64: "<i8"}


class _RawCuda:
    """Minimal ``__cuda_array_interface__`` carrier so torch can wrap a cudaMalloc'd address."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


def wrap_device_memory(ptr: int, nbytes: int, device: torch.device) -> torch.Tensor:
    return torch.as_tensor(_RawCuda(ptr, nbytes), device=device)


class SymmetricBuffer:
    def __init__(self, nbytes: int, device, group=None, zero: bool = False):
        self.device = torch.device(device)
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        out = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            check(lib().rpeg_symm_alloc(self.nbytes, ctypes.byref(out)), "rpeg_symm_alloc")
            self.ptr = int(out.value)
            self.bytes_view = wrap_device_memory(self.ptr, self.nbytes, self.device)
            if zero:
                self.bytes_view.zero_()
            self.peer_ptrs: List[int] = [0] * self.world
            self.peer_ptrs[self.rank] = self.ptr
            self._opened: List[int] = []
            if self.world > 1:
                handle = (ctypes.c_ubyte * 64)()
                check(lib().rpeg_ipc_export(self.ptr, handle), "rpeg_ipc_export")
                handles: List[Optional[bytes]] = [None] * self.world
                dist.all_gather_object(handles, bytes(handle), group=group)
                for r, h in enumerate(handles):
                    if r == self.rank:
                        continue
                    buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                    p = ctypes.c_void_p()
                    check(lib().rpeg_ipc_open(buf, ctypes.byref(p)), "rpeg_ipc_open")
                    self.peer_ptrs[r] = int(p.value)
                    self._opened.append(int(p.value))
                torch.cuda.synchronize(self.device)
                dist.barrier(group=group)
        self._ptr_array = (ctypes.c_void_p * self.world)(*self.peer_ptrs)

    def tensor(self, dtype: torch.dtype, numel: Optional[int] = None, byte_offset: int = 0) -> torch.Tensor:
        item = torch.empty(0, dtype=dtype).element_size()
        n = (self.nbytes - byte_offset) // item if numel is None else numel
        return self.bytes_view[byte_offset:byte_offset + n * item].view(dtype)

    def ptr_array(self, byte_offset: int = 0):
        """ctypes ``void*[world]`` of the peers' addresses (optionally displaced by ``byte_offset``)."""
        if byte_offset == 0:
            return self._ptr_array
        return (ctypes.c_void_p * self.world)(*[p + byte_offset for p in self.peer_ptrs])

    def close(self) -> None:
        for p in self._opened:
            lib().rpeg_ipc_close(p)
        self._opened = []
        if self.ptr:
            self.bytes_view = None
            lib().rpeg_symm_free(self.ptr)
            self.ptr = 0


class SignalPad(SymmetricBuffer):
    """64 flag slots x 8 ranks of uint32 followed by a float payload area (see ``flag_barrier_kernel``)."""

    FLAG_WORDS = 1024
    PAYLOAD_WORDS = 1024

    def __init__(self, device, group=None):
        super().__init__((self.FLAG_WORDS + self.PAYLOAD_WORDS) * 4, device, group, zero=True)
        self.epochs = [0] * 64
