"""One-shot all-reduce fused with the residual add and the next normalisation
(``csrc/allreduce.cu``): the collective of tensor-parallel decoding.  ``backend="fused"`` reads
every rank's partial result through NVLink peer mappings inside one kernel whose parameters never
change between calls (so it can be replayed from a CUDA graph); ``backend="nccl"`` composes
``all_reduce`` with the stand-alone kernels and is the baseline and the path of CPU ranks.  The
reference has no collective of any kind."""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import norm as N


class FusedAllReduce:
    def __init__(self, group, device, max_rows: int, hidden: int, backend: Optional[str] = None,
                 wait_limit_ms: float = 5000.0, dtype=torch.bfloat16) -> None:
        self.group = group
        self.device = torch.device(device)
        self.rank = dist.get_rank(group) if group is not None else 0
        self.tp = dist.get_world_size(group) if group is not None else 1
        if backend is None:
            backend = "fused" if self.device.type == "cuda" and self.tp > 1 else "nccl"
        self.backend = backend
        self.max_rows, self.H = max_rows, hidden
        self.limit_ns = int(wait_limit_ms * 1e6)
        self._turn = 0
        if backend == "fused":
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
