"""All-to-all of equal blocks between the ranks of a group.

``backend="p2p"``: the send blocks are written into a symmetric buffer and every rank pulls its
block from each peer over NVLink with a copy kernel (signal pads say when a buffer may be read and
when it may be overwritten); ``backend="collective"``: ``all_to_all_single`` on NCCL, and on CPU
ranks an all-gather based restatement (Gloo has no all-to-all for every build).  Used by Ulysses
sequence parallelism; the mixture-of-experts exchange does not come through here, it is fused into
the expert GEMMs.  The reference has no communication layer at all.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist


class AllToAll:
    def __init__(self, group, device, backend: Optional[str] = None,
                 wait_limit_ms: float = 5000.0) -> None:
        self.group = group
        self.device = torch.device(device)
        self.rank = dist.get_rank(group) if group is not None else 0
        self.world = dist.get_world_size(group) if group is not None else 1
        if backend is None:
            backend = "p2p" if self.device.type == "cuda" and self.world > 1 else "collective"
        self.backend = backend
        self.limit_ms = wait_limit_ms
        self._sym = None
        self._epoch = 0
        self.pad = None
        if backend == "p2p":
            from .symm import SignalPad
            self.pad = SignalPad(2, group, self.device, wait_limit_ms)

    def exchange(self, send: torch.Tensor) -> torch.Tensor:
        """``send [world, ...]`` (block ``d`` goes to rank ``d``) -> ``recv [world, ...]`` (block
        ``s`` came from rank ``s``)."""
        w = self.world
        assert send.shape[0] == w
        if w == 1:
            return send
        send = send.contiguous()
        recv = torch.empty_like(send)
        if self.backend != "p2p":
            if send.is_cuda:
                dist.all_to_all_single(recv, send, group=self.group)
            else:
                parts = [torch.empty_like(send) for _ in range(w)]
                dist.all_gather(parts, send, group=self.group)
                for s in range(w):
                    recv[s].copy_(parts[s][self.rank])
            return recv
        from ..ops import _lib
        from .symm import SymmetricBuffer
        nbytes = send.numel() * send.element_size()
        blk = nbytes // w
        if blk % 16:
            raise ValueError("all-to-all blocks must be multiples of 16 bytes")
        if self._sym is None or self._sym.nbytes < nbytes:
            self._sym = SymmetricBuffer(nbytes, self.group, self.device)
            self._epoch = 0
        if self._epoch > 0:
            self.pad.wait(1, self._epoch)             # everyone has pulled my previous blocks
        self._epoch += 1
        self._sym.local[:nbytes].copy_(send.view(-1).view(torch.uint8))
        self.pad.signal(0, self._epoch)
        self.pad.wait(0, self._epoch)                 # everyone's blocks are published
        rbytes = recv.view(-1).view(torch.uint8)
        for t in range(w):
            s = (self.rank + t) % w                   # stagger the peers
            rc = _lib.lib().cb_peer_copy(ctypes.c_void_p(self._sym.ptrs[s] + self.rank * blk),
                                         ctypes.c_void_p(rbytes.data_ptr() + s * blk),
                                         ctypes.c_size_t(blk), 0, _lib.stream_ptr())
            _lib.check_rc(rc, "cb_peer_copy")
        self.pad.signal(1, self._epoch)
        return recv
