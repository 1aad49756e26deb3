"""One-shot all-reduce fused with the residual add and the next normalisation
(``csrc/allreduce.cu``): the collective of tensor-parallel decoding.  ``backend="nvls"`` reduces
in the NVLink switch: each rank pulls its share of the rows with ``multimem.ld_reduce`` from a
multicast mapping of all ranks' partial buffers and writes the finished rows to every rank with
``multimem.st``; ``backend="fused"`` reads every rank's partial result through plain NVLink peer
mappings.  Both are one kernel whose parameters never change between calls (so it can be replayed
from a CUDA graph).  ``backend=None`` picks ``nvls`` where the devices support multicast objects
(``COEUS_NVLS=0`` switches that off), else ``fused``.  ``backend="nccl"`` composes
``all_reduce`` with the stand-alone kernels and is the baseline and the path of CPU ranks.  The
reference has no collective of any kind."""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import norm as N


class FusedAllReduce:
    def __init__(self, group, device, max_rows: int, hidden: int, backend: Optional[str] = None,
                 wait_limit_ms: float = 5000.0, dtype=torch.bfloat16,
                 one_shot: Optional[bool] = None) -> None:
        """``one_shot`` (``nvls`` only): every rank reduces all rows for itself with
        ``multimem.ld_reduce`` and stores locally -- one counter round trip instead of two, at
        ``tp`` times the switch traffic; the default (``COEUS_NVLS_ONESHOT``, else off) is the
        two-phase form in which a rank handles ``1/tp`` of the rows and broadcasts them."""
        self.group = group
        self.device = torch.device(device)
        self.rank = dist.get_rank(group) if group is not None else 0
        self.tp = dist.get_world_size(group) if group is not None else 1
        if backend is None:
            backend = "fused" if self.device.type == "cuda" and self.tp > 1 else "nccl"
            if backend == "fused" and os.environ.get("COEUS_NVLS", "1") != "0":
                from .symm import multicast_supported
                if multicast_supported(self.device):
                    backend = "nvls"
        self.backend = backend
        self.max_rows, self.H = max_rows, hidden
        self.limit_ns = int(wait_limit_ms * 1e6)
        self._turn = 0
        if one_shot is None:
            one_shot = os.environ.get("COEUS_NVLS_ONESHOT", "0") == "1"
        self.one_shot = bool(one_shot)
        if backend == "nvls":
            from .symm import MulticastBuffer
            n = max_rows * hidden * 2                 # bytes of one [max_rows, H] bf16 buffer
            self._stride = (n + 255) // 256 * 256
            # one allocation: 2 partial buffers, 2 x outputs, 2 n outputs, then the counters
            self._mc = MulticastBuffer(6 * self._stride + 256, group, self.device)
            self._mc.local.zero_()
            view = lambda i: self._mc.view(torch.bfloat16, i * self._stride,   # noqa: E731
                                           max_rows * hidden).view(max_rows, hidden)
            self.parts = [view(0), view(1)]
            self._x = [view(2), view(3)]
            self._n = [view(4), view(5)]
            self._state = torch.zeros(2, dtype=torch.int64, device=self.device)
            torch.cuda.synchronize(self.device)
            dist.barrier(group=group)
        elif backend == "fused":
            from .symm import SymmetricBuffer
            n = max_rows * hidden
            self._sym = [SymmetricBuffer(n * 2, group, self.device) for _ in range(2)]
            self.parts = [s.view(torch.bfloat16, 0, n).view(max_rows, hidden) for s in self._sym]
            self._flags = SymmetricBuffer(256, group, self.device)
            self._flags.local.zero_()
            self._state = torch.zeros(2, dtype=torch.int64, device=self.device)
            torch.cuda.synchronize(self.device)
            dist.barrier(group=group)
            self._part_ptrs = [s.ptr_array() for s in self._sym]
            self._flag_ptrs = self._flags.ptr_array()
        else:
            self.parts = [torch.empty((max_rows, hidden), dtype=dtype, device=self.device)
                          for _ in range(2)]

    def next_part(self, rows: int) -> torch.Tensor:
        """The buffer the next partial result has to be written into (``[rows, H]`` view)."""
        return self.parts[self._turn][:rows]

    def reduce(self, rows: int, resid: Optional[torch.Tensor], scale: Optional[torch.Tensor],
               bias: Optional[torch.Tensor], rms: bool, eps: float
               ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """Sum of all ranks' ``next_part`` buffers (+ ``resid``) and, when ``scale`` is given,
        its normalisation: ``(x, n)``."""
        turn = self._turn
        self._turn ^= 1
        part = self.parts[turn][:rows]
        if self.backend == "nvls":
            # results land in this rank's copy of the symmetric output buffers (every rank's
            # rows are written by their owner through the multicast mapping); the views stay
            # valid until the call after next
            mc, sd = self._mc, self._stride
            x = self._x[turn][:rows]
            n = self._n[turn][:rows] if scale is not None else None
            st = _lib.status_buffer(self.device)
            out_base = mc.local_ptr if self.one_shot else mc.mc_ptr
            rc = _lib.lib().cb_ar_multimem(
                ctypes.c_void_p(mc.mc_ptr + turn * sd), ctypes.c_void_p(out_base + (2 + turn) * sd),
                ctypes.c_void_p(out_base + (4 + turn) * sd) if scale is not None else None,
                _lib.ptr(resid), ctypes.c_void_p(mc.mc_ptr + 6 * sd),
                ctypes.c_void_p(mc.local_ptr + 6 * sd), _lib.ptr(self._state), _lib.ptr(scale),
                _lib.ptr(bias), self.tp, self.rank, rows, self.H, int(rms), ctypes.c_float(eps),
                ctypes.c_ulonglong(self.limit_ns), _lib.ptr(st), int(self.one_shot),
                _lib.stream_ptr())
            _lib.check_rc(rc, "cb_ar_multimem")
            return x, n
        if self.backend != "fused":
            x = part.clone()
            if self.tp > 1:
                dist.all_reduce(x, group=self.group)
            if resid is not None:
                x = (x.float() + resid.float()).to(part.dtype)
            n = None
            if scale is not None:
                n, _, _ = N.norm_fwd(x, scale, bias, eps, rms)
            return x, n
        x = torch.empty((rows, self.H), dtype=torch.bfloat16, device=self.device)
        n = torch.empty_like(x) if scale is not None else None
        st = _lib.status_buffer(self.device)
        rc = _lib.lib().cb_ar_resid_norm(
            self._part_ptrs[turn], self._flag_ptrs, ctypes.c_void_p(self._flags.local_ptr),
            _lib.ptr(self._state), _lib.ptr(resid), _lib.ptr(x), _lib.ptr(scale), _lib.ptr(bias),
            _lib.ptr(n), self.tp, self.rank, rows, self.H, int(rms), ctypes.c_float(eps),
            ctypes.c_ulonglong(self.limit_ns), _lib.ptr(st), _lib.stream_ptr())
        _lib.check_rc(rc, "cb_ar_resid_norm")
        return x, n


    def close(self) -> None:
        """Release the symmetric memory (collective: no rank may still be using it)."""
        if self.backend == "nvls" and getattr(self, "_mc", None) is not None:
            self.parts, self._x, self._n = [], [], []
            self._mc.close()
            self._mc = None


class GreedySelect:
    """Arg-max over a vocabulary split across ranks (``csrc/allreduce.cu: greedy_select``): each
    rank pushes one (value, index) pair per sequence into every peer's table over NVLink and picks
    the best of all ranks -- no library collective, fixed launch parameters (graph-replayable)."""

    def __init__(self, group, device, max_batch: int, wait_limit_ms: float = 5000.0) -> None:
        from .symm import SymmetricBuffer
        self.group, self.device = group, torch.device(device)
        self.rank, self.tp = dist.get_rank(group), dist.get_world_size(group)
        self.max_batch = max_batch
        self.limit_ns = int(wait_limit_ms * 1e6)
        n = self.tp * max_batch * 8
        self._pairs = SymmetricBuffer(n, group, self.device)
        self._flags = SymmetricBuffer(n, group, self.device)
        self._flags.local.zero_()
        self._state = torch.zeros(2, dtype=torch.int64, device=self.device)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)
        self._pair_ptrs, self._flag_ptrs = self._pairs.ptr_array(), self._flags.ptr_array()
        self._batch = None

    def select(self, logits_l: torch.Tensor, valid: int, col0: int) -> torch.Tensor:
        """``logits_l [B, >=valid]`` bf16 (this rank's columns, the first ``valid`` compete,
        column 0 is token ``col0``) -> chosen token ids ``[B]`` int64, identical on all ranks."""
        B = logits_l.shape[0]
        if self._batch is None:
            self._batch = B          # the slot layout [tp][B] is fixed by the first call
        if B != self._batch or B > self.max_batch:
            raise ValueError("GreedySelect is bound to the batch size of its first call")
        out = torch.empty(B, dtype=torch.int64, device=self.device)
        st = _lib.status_buffer(self.device)
        rc = _lib.lib().cb_greedy_select(
            _lib.ptr(logits_l), logits_l.stride(0), valid, col0, self._pair_ptrs, self._flag_ptrs,
            _lib.ptr(self._state), _lib.ptr(out), self.tp, self.rank, B,
            ctypes.c_ulonglong(self.limit_ns), _lib.ptr(st), _lib.stream_ptr())
        _lib.check_rc(rc, "cb_greedy_select")
        return out
