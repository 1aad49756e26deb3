"""Symmetric buffers over NVLink peer memory.

Every rank allocates a buffer of the same size with ``cudaMalloc`` (through the kernel library),
exports it with CUDA IPC, and maps every peer's buffer, so kernels can address "the same offset
on rank r".  The local buffer is exposed as a ``torch`` tensor (zero-copy through
``__cuda_array_interface__``); peers are raw device pointers handed to the kernels.  Signal flags
(64-bit epochs) live in one such buffer.  The reference has no communication layer at all
(single process); this is the substrate the fused compute+collective kernels stand on.

:class:`MulticastBuffer` is the same thing built on the virtual-memory-management API
(``csrc/vmm.cu``): allocations made with ``cuMemCreate``, exchanged as file descriptors over Unix
sockets, mapped on every rank, and bound to one NVLink multicast object (NVLS), whose mapping
``mc_ptr`` addresses "this offset on all ranks at once" -- what ``multimem.ld_reduce``,
``multimem.st`` and ``multimem.red`` operate on.
"""
from __future__ import annotations

import atexit
import ctypes
import os
import socket
import threading
import uuid
import weakref
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


def exchange_fds(group, fds: List[int]) -> List[List[int]]:
    """Every rank offers a list of file descriptors; returns, by rank, the descriptors received
    from that rank (duplicates valid in this process; the caller closes them).  Descriptors
    travel as ancillary data over Unix-domain sockets in the abstract namespace, so all ranks
    must run on one host -- which peer memory over NVLink requires anyway."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    name = "\0coeus-fd-%d-%s" % (os.getpid(), uuid.uuid4().hex)
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    srv.bind(name)
    srv.listen(world)
    srv.settimeout(120.0)
    names: List[Optional[str]] = [None] * world
    dist.all_gather_object(names, name, group=group)
    errors: List[BaseException] = []

    def serve() -> None:
        try:
            for _ in range(world - 1):
                conn, _addr = srv.accept()
                with conn:
                    socket.send_fds(conn, [b"f"], list(fds))
        except BaseException as e:      # surfaced below
            errors.append(e)

    th = threading.Thread(target=serve, name="coeus-fd-server", daemon=True)
    th.start()
    out: List[List[int]] = [[] for _ in range(world)]
    for r in range(world):
        if r == rank:
            out[r] = [os.dup(fd) for fd in fds]
            continue
        with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as c:
            c.settimeout(120.0)
            c.connect(names[r])
            _msg, got, _flags, _addr = socket.recv_fds(c, 16, 8)
            out[r] = list(got)
    th.join(timeout=120.0)
    srv.close()
    if errors:
        raise CommError.mismatch(f"descriptor exchange failed: {errors[0]!r}")
    return out


_LIVE_MULTICAST: "weakref.WeakSet[MulticastBuffer]" = weakref.WeakSet()


def _close_all_multicast() -> None:
    for b in list(_LIVE_MULTICAST):
        b.close()


atexit.register(_close_all_multicast)


def multicast_supported(device) -> bool:
    """Whether the device can take part in an NVLink multicast object (NVLS)."""
    with torch.cuda.device(device):
        return _lib.lib().cb_multicast_supported() == 1


class MulticastBuffer:
    """A symmetric allocation that is also bound to an NVLink multicast object.

    ``local`` is this rank's memory (uint8 tensor), ``ptrs[r]`` the mapping of rank ``r``'s
    memory in this process (plain peer loads / stores), ``mc_ptr`` the multicast mapping.
    Sizes are rounded up to the granularity of the allocator and of multicast objects (2 MiB or
    more), so many logical buffers should share one allocation (``view`` / byte offsets).
    ``close()`` unbinds and frees in the order the driver wants; it also runs at interpreter
    exit, because a process must not end with its memory still bound to the multicast object.
    """

    def __init__(self, nbytes: int, group, device: torch.device) -> None:
        self.group, self.device = group, torch.device(device)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        lib = _lib.lib()
        for fn in (lib.cb_vmm_granularity,):
            fn.restype = ctypes.c_size_t
        self._mem = self._mc = None
        self._peers: List[int] = []
        with torch.cuda.device(self.device):
            if lib.cb_multicast_supported() != 1:
                raise CommError.mismatch("this device does not support NVLink multicast objects")
            g_mem = lib.cb_vmm_granularity(0, self.world)
            g_mc = lib.cb_vmm_granularity(1, self.world)
            if not g_mem or not g_mc:
                raise CommError.mismatch("could not query the allocation granularity")
            gran = max(g_mem, g_mc)
            self.nbytes = (nbytes + gran - 1) // gran * gran
            mem, va = ctypes.c_void_p(), ctypes.c_void_p()
            rc = lib.cb_vmm_alloc(ctypes.c_size_t(self.nbytes), ctypes.byref(mem), ctypes.byref(va))
            if rc != 0:
                raise ResourceError.exhausted("device memory (cuMemCreate)", 0, self.nbytes)
            self._mem, self.local_ptr = mem, va.value
            fd = ctypes.c_int(-1)
            if lib.cb_vmm_export_fd(self._mem, ctypes.byref(fd)) != 0:
                raise CommError.mismatch("cuMemExportToShareableHandle failed")
            mine = [fd.value]
            if self.rank == 0:
                mc, mfd = ctypes.c_void_p(), ctypes.c_int(-1)
                rc = lib.cb_mc_create(self.world, ctypes.c_size_t(self.nbytes), ctypes.byref(mc),
                                      ctypes.byref(mfd))
                if rc != 0:
                    raise CommError.mismatch(f"cuMulticastCreate failed ({rc})")
                self._mc = mc
                mine.append(mfd.value)
            got = exchange_fds(group, mine)
            for f in mine:
                os.close(f)
            self.ptrs: List[int] = []
            for r in range(self.world):
                if r == self.rank:
                    self.ptrs.append(self.local_ptr)
                else:
                    h, p = ctypes.c_void_p(), ctypes.c_void_p()
                    rc = lib.cb_vmm_import(got[r][0], ctypes.c_size_t(self.nbytes),
                                           ctypes.byref(h), ctypes.byref(p))
                    if rc != 0:
                        raise CommError.mismatch(f"import of rank {r}'s memory failed ({rc})")
                    self._peers.append(h)
                    self.ptrs.append(p.value)
            if self.rank != 0:
                mc = ctypes.c_void_p()
                rc = lib.cb_mc_import(got[0][1], ctypes.c_size_t(self.nbytes), ctypes.byref(mc))
                if rc != 0:
                    raise CommError.mismatch(f"import of the multicast object failed ({rc})")
                self._mc = mc
            for fds in got:
                for f in fds:
                    os.close(f)
            if lib.cb_mc_add_device(self._mc) != 0:
                raise CommError.mismatch("cuMulticastAddDevice failed")
            dist.barrier(group=group)          # every device is part of the team before binding
            mcva = ctypes.c_void_p()
            rc = lib.cb_mc_bind_map(self._mc, self._mem, ctypes.byref(mcva))
            if rc != 0:
                raise CommError.mismatch(f"cuMulticastBindMem / mapping failed ({rc})")
            self.mc_ptr = mcva.value
        self._holder = _RawCudaBuffer(self.local_ptr, self.nbytes)
        self.local = torch.as_tensor(self._holder, device=self.device)
        _LIVE_MULTICAST.add(self)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)              # every rank has bound its memory

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
        """Unbind from the multicast object and free everything (idempotent).  Collective in
        spirit: no rank may still be running kernels that touch the buffer."""
        lib = _lib.lib()
        if self._mc is None and self._mem is None:
            return
        try:
            torch.cuda.synchronize(self.device)
        except Exception:
            pass
        with torch.cuda.device(self.device):
            if self._mc is not None:
                lib.cb_mc_release(self._mc)
                self._mc = None
            for h in self._peers:
                lib.cb_vmm_release(h)
            self._peers = []
            if self._mem is not None:
                lib.cb_vmm_release(self._mem)
                self._mem = None
        self.local = None
        _LIVE_MULTICAST.discard(self)


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
