"""Symmetric buffers across the ranks of one node: same size on every rank, every rank holds a
device pointer to every peer's copy (CUDA IPC over NVLink peer access).

``SymmetricBuffer`` is allocated collectively; ``local`` is a normal torch tensor over this rank's
memory and ``peer_ptrs`` are raw device addresses (this rank's own included, in rank order) that the
fused kernels take. ``SignalPad`` is a small zero-initialised symmetric buffer with flag slots and
a float payload area used by the device-side barrier.

Every buffer is allocated with ``GUARD`` bytes of a fixed pattern in front of and behind the usable range. Kernels
of ANY rank write into these buffers through raw addresses, so an index error in a fused kernel lands in a
neighbouring allocation without a fault; ``check_canaries()`` reads the guard bytes of all live buffers back and
raises when one changed (tests and ``parallel/selftest.py`` call it after every fused path).

Handles travel over ``torch.distributed`` object collectives (NCCL/Gloo group of the job), so this
layer needs no MPI, UCX or filesystem rendezvous. The reference moves such tensors between
processes through pickled CUDA-IPC storages and ad-hoc NCCL groups
(RPEG/runtime/semantic_worker.py:9840-10028, 11281-11365).
"""
from __future__ import annotations

import contextlib
import ctypes
import weakref
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops._lib import check, lib

GUARD = 256            # bytes of canary pattern on each side of a symmetric buffer (keeps the 256-byte alignment)
CANARY = 0xA5
_LIVE: "weakref.WeakSet[SymmetricBuffer]" = weakref.WeakSet()


class SymmetricMemoryCorruption(RuntimeError):
    pass


def check_canaries() -> int:
    """Read back the guard bytes of every live symmetric buffer of this process; raises on the first buffer whose
    guards changed (some kernel, local or on a peer, wrote outside the buffer). Returns the number of buffers checked."""
    n = 0
    for buf in list(_LIVE):
        bad = buf.corrupted_guards()
        if bad:
            raise SymmetricMemoryCorruption(f"symmetric buffer of {buf.nbytes} bytes at {buf.ptr:#x} on rank {buf.rank}: "
                                            f"guard bytes overwritten {bad}")
        n += 1
    return n


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
        with (torch.cuda.device(self.device) if self.device.type == "cuda" else contextlib.nullcontext()):
            check(lib().rpeg_symm_alloc(self.nbytes + 2 * GUARD, ctypes.byref(out)), "rpeg_symm_alloc")
            self._base = int(out.value)
            self.ptr = self._base + GUARD
            raw = wrap_device_memory(self._base, self.nbytes + 2 * GUARD, self.device)
            self._guards = (raw[:GUARD], raw[GUARD + self.nbytes:])
            for g in self._guards:
                g.fill_(CANARY)
            self.bytes_view = raw[GUARD:GUARD + self.nbytes]
            if zero:
                self.bytes_view.zero_()
            self.peer_ptrs: List[int] = [0] * self.world
            self.peer_ptrs[self.rank] = self.ptr
            self._opened: List[int] = []
            if self.world > 1:
                handle = (ctypes.c_ubyte * 64)()
                check(lib().rpeg_ipc_export(self._base, handle), "rpeg_ipc_export")
                handles: List[Optional[bytes]] = [None] * self.world
                dist.all_gather_object(handles, bytes(handle), group=group)
                for r, h in enumerate(handles):
                    if r == self.rank:
                        continue
                    buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                    p = ctypes.c_void_p()
                    check(lib().rpeg_ipc_open(buf, ctypes.byref(p)), "rpeg_ipc_open")
                    self.peer_ptrs[r] = int(p.value) + GUARD
                    self._opened.append(int(p.value))
                torch.cuda.synchronize(self.device)
                dist.barrier(group=group)
        self._ptr_array = (ctypes.c_void_p * self.world)(*self.peer_ptrs)
        _LIVE.add(self)

    def corrupted_guards(self) -> List[str]:
        """``["front+offset", "back+offset"]`` for each guard region with a changed byte (empty when intact)."""
        if not self.ptr:
            return []
        out = []
        for name, g in zip(("front", "back"), self._guards):
            bad = (g != CANARY).nonzero()
            if bad.numel():
                out.append(f"{name}+{int(bad[0])}")
        return out

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
            _LIVE.discard(self)
            self.bytes_view = None
            self._guards = ()
            lib().rpeg_symm_free(self._base)
            self.ptr = 0


class SignalPad(SymmetricBuffer):
    """64 flag slots x 8 ranks of uint32 followed by a float payload area (see ``flag_barrier_kernel``)."""

    FLAG_WORDS = 1024
    PAYLOAD_WORDS = 1024

    def __init__(self, device, group=None):
        super().__init__((self.FLAG_WORDS + self.PAYLOAD_WORDS) * 4, device, group, zero=True)
        self.epochs = [0] * 64
