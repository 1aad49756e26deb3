"""Symmetric buffers over NVLink peer memory.

Every rank allocates a buffer of the same size with ``cudaMalloc`` (through the kernel library),
exports it with CUDA IPC, and maps every peer's buffer, so kernels can address "the same offset
on rank r".  The local buffer is exposed as a ``torch`` tensor (zero-copy through
``__cuda_array_interface__``); peers are raw device pointers handed to the kernels.  Signal flags
(64-bit epochs) live in one such buffer.  The reference has no communication layer at all
(single process); this is the substrate the fused compute+collective kernels stand on.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..foundation.error import CommError, ResourceError
from ..ops import _lib


class _RawCudaBuffer:
    def __init__(self, ptr: int, nbytes: int) -> None:
        self.ptr, self.nbytes = ptr, nbytes
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1",
                                         "data": (ptr, False), "version": 3}


class SymmetricBuffer:
    """One symmetric allocation: ``local`` (uint8 tensor), ``ptrs[r]`` device pointers by rank."""

    def __init__(self, nbytes: int, group, device: torch.device) -> None:
        self.group = group
        self.device = device
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.nbytes = (nbytes + 255) // 256 * 256
        lib = _lib.lib()
        out = ctypes.c_void_p()
        with torch.cuda.device(device):
            rc = lib.cb_symm_alloc(ctypes.c_size_t(self.nbytes), ctypes.byref(out))
        if rc != 0:
            raise ResourceError.exhausted("device memory", 0, self.nbytes)
        self.local_ptr = out.value
        self._holder = _RawCudaBuffer(self.local_ptr, self.nbytes)
        self.local = torch.as_tensor(self._holder, device=device)
        handle = (ctypes.c_ubyte * 64)()
        if lib.cb_ipc_get_handle(ctypes.c_void_p(self.local_ptr), handle) != 0:
            raise CommError.mismatch("cudaIpcGetMemHandle failed")
        handles: List[Optional[bytes]] = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.ptrs: List[int] = []
        self._opened: List[int] = []
        with torch.cuda.device(device):
            for r, h in enumerate(handles):
                if r == self.rank:
                    self.ptrs.append(self.local_ptr)
                    continue
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                p = ctypes.c_void_p()
                rc = lib.cb_ipc_open(buf, ctypes.byref(p))
                if rc != 0:
                    raise CommError.mismatch(f"cudaIpcOpenMemHandle for rank {r} failed ({rc})")
                self.ptrs.append(p.value)
                self._opened.append(p.value)
        dist.barrier(group=group)

    def ptr_array(self, byte_offset: int = 0):
        arr = (ctypes.c_void_p * self.world)()
        for i, p in enumerate(self.ptrs):
            arr[i] = p + byte_offset
        return arr

    def view(self, dtype: torch.dtype, byte_offset: int = 0, numel: Optional[int] = None) -> torch.Tensor:
        t = self.local[byte_offset:]
        item = torch.empty((), dtype=dtype).element_size()
        if numel is not None:
            t = t[: numel * item]
        return t.view(dtype)

    def close(self) -> None:
        lib = _lib.lib()
        for p in self._opened:
            lib.cb_ipc_close(ctypes.c_void_p(p))
        self._opened = []


class SignalPad:
    """``slots x world`` 64-bit flags per rank; ``signal(slot, value)`` writes this rank's flag in
    every peer's pad, ``wait(slot, value)`` blocks the stream (bounded) until all ranks' flags in
    the local pad reached ``value``."""

    def __init__(self, slots: int, group, device: torch.device, limit_ms: float = 2000.0) -> None:
        self.slots = slots
        self.buf = SymmetricBuffer(slots * dist.get_world_size(group) * 8, group, device)
        self.world, self.rank = self.buf.world, self.buf.rank
        self.device = device
        self.limit_ns = int(limit_ms * 1e6)
        self._ptrs = self.buf.ptr_array()

    def signal(self, slot: int, value: int) -> None:
        rc = _lib.lib().cb_signal_peers(self._ptrs, slot, self.world, self.rank,
                                        ctypes.c_ulonglong(value), _lib.stream_ptr())
        _lib.check_rc(rc, "cb_signal_peers")

    def wait(self, slot: int, value: int) -> None:
        st = _lib.status_buffer(self.device)
        rc = _lib.lib().cb_wait_flags(ctypes.c_void_p(self.buf.local_ptr), slot, self.world,
                                      ctypes.c_ulonglong(value), ctypes.c_ulonglong(self.limit_ns),
                                      _lib.ptr(st), _lib.stream_ptr())
        _lib.check_rc(rc, "cb_wait_flags")

    def barrier(self, slot: int, value: int) -> None:
        self.signal(slot, value)
        self.wait(slot, value)


class OffsetAllocator:
    """First-fit allocator over ``[0, size)`` with coalescing free list: the bookkeeping of a
    symmetric heap.  Pure host logic; all ranks that make the same sequence of calls get the same
    offsets, which is what makes "the same offset on rank r" meaningful."""

    def __init__(self, size: int, alignment: int = 256) -> None:
        self.size, self.alignment = size, alignment
        self.free: List[List[int]] = [[0, size]]          # sorted [start, end) holes
        self.live = {}                                     # start -> end
        self.peak = 0

    def alloc(self, nbytes: int) -> int:
        a = self.alignment
        need = max(a, (nbytes + a - 1) // a * a)
        for hole in self.free:
            if hole[1] - hole[0] >= need:
                start = hole[0]
                hole[0] += need
                if hole[0] == hole[1]:
                    self.free.remove(hole)
                self.live[start] = start + need
                self.peak = max(self.peak, self.used())
                return start
        raise ResourceError.exhausted("symmetric heap", self.size - self.used(), need)

    def release(self, start: int) -> None:
        end = self.live.pop(start)
        holes = sorted(self.free + [[start, end]])
        merged: List[List[int]] = []
        for h in holes:
            if merged and merged[-1][1] == h[0]:
                merged[-1][1] = h[1]
            else:
                merged.append(h)
        self.free = merged

    def used(self) -> int:
        return sum(e - s for s, e in self.live.items())


class SymmetricRegion:
    """A piece of a :class:`SymmetricHeap`: ``local`` bytes of this rank, ``ptrs[r]`` by rank."""

    def __init__(self, heap: "SymmetricHeap", offset: int, nbytes: int) -> None:
        self.heap, self.offset, self.nbytes = heap, offset, nbytes
        self.local = heap.buf.local[offset:offset + nbytes]
        self.local_ptr = heap.buf.local_ptr + offset
        self.ptrs = [p + offset for p in heap.buf.ptrs]

    def ptr_array(self, byte_offset: int = 0):
        return self.heap.buf.ptr_array(self.offset + byte_offset)

    def view(self, dtype: torch.dtype, numel: Optional[int] = None) -> torch.Tensor:
        return self.heap.buf.view(dtype, self.offset,
                                  numel if numel is not None else
                                  self.nbytes // torch.empty((), dtype=dtype).element_size())

    def free(self) -> None:
        self.heap.alloc_state.release(self.offset)


class SymmetricHeap:
    """One peer-mapped allocation per rank, sub-allocated on the host: many symmetric tensors
    cost one IPC exchange, and every region's offset is the same on all ranks because all ranks
    allocate in the same order (a collective convention, like the order of collectives)."""

    def __init__(self, nbytes: int, group, device: torch.device, alignment: int = 256) -> None:
        self.buf = SymmetricBuffer(nbytes, group, device)
        self.alloc_state = OffsetAllocator(self.buf.nbytes, alignment)

    def alloc(self, nbytes: int) -> SymmetricRegion:
        return SymmetricRegion(self, self.alloc_state.alloc(nbytes), nbytes)

    def close(self) -> None:
        self.buf.close()
