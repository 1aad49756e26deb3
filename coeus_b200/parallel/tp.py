"""Tensor parallelism with sequence-parallel activations (Megatron style), built on two fused
kernels of ``csrc/gemm.cu``:

* ``ag_gemm``: all-gather of the per-rank row shards ``[T/tp, K]`` -> column-parallel GEMM
  (QKV; gate/up).  Every rank keeps one symmetric ``[T, K]`` buffer, writes its own rows, and the
  GEMM kernel's pull warps fetch the other ranks' rows over NVLink (plain peer loads) into the
  local copy while the tensor cores already work on the rows that are there; the gathered copy
  stays for the weight-gradient GEMM.
* ``gemm_rs``: row-parallel GEMM (O projection; down projection) -> reduce-scatter along the
  rows.  The epilogue pushes every tile of partial sums into the owner's receive slot with
  coalesced peer stores; the owner sums the ``tp`` slots (+ residual) in a small kernel.

``backend="nccl"`` composes the same results from ``torch.distributed`` collectives and the
plain GEMM: it is the baseline the fused kernels are measured against, and the path CPU ranks
(Gloo) take.  The reference has no parallelism of any kind.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ..foundation.error import ProcessingError
from ..ops import _lib
from ..ops import gemm as G


class _CommArgs(ctypes.Structure):
    _fields_ = [("comm", ctypes.c_int), ("tp", ctypes.c_int), ("rank", ctypes.c_int),
                ("rows_per_shard", ctypes.c_int), ("ag_src", ctypes.c_void_p * 8),
                ("ag_flags", ctypes.c_void_p), ("ag_epoch", ctypes.c_uint),
                ("peer_flags", ctypes.c_void_p), ("peer_expect", ctypes.c_ulonglong),
                ("wait_limit_ns", ctypes.c_ulonglong), ("rs_dst", ctypes.c_void_p * 8),
                ("rs_ld", ctypes.c_int)]


class _Site:
    """Buffers and epoch of one collective call site (e.g. "layer-independent QKV gather")."""

    def __init__(self) -> None:
        self.epoch = 0


class TensorParallel:
    def __init__(self, group, device, backend: Optional[str] = None,
                 wait_limit_ms: float = 5000.0, max_sites: int = 16) -> None:
        self.group = group
        self.device = torch.device(device)
        self.rank = dist.get_rank(group)
        self.tp = dist.get_world_size(group)
        if backend is None:
            backend = "fused" if self.device.type == "cuda" and self.tp > 1 else "nccl"
        if backend not in ("fused", "nccl"):
            raise ProcessingError.invalid_input(f"unknown tensor-parallel backend '{backend}'")
        if self.tp > 8 and backend == "fused":
            raise ProcessingError.limit_exceeded("tensor-parallel ranks", 8, self.tp)
        self.backend = backend
        self.limit_ns = int(wait_limit_ms * 1e6)
        self.sites: Dict[str, _Site] = {}
        self.max_sites = max_sites
        self.pad = None
        if backend == "fused":
            from .symm import SignalPad
            # per site: slot 2i = "data written / pushed", slot 2i+1 = "data consumed"
            self.pad = SignalPad(2 * max_sites, group, self.device, wait_limit_ms)

    # ------------------------------------------------------------------ helpers
    def _site(self, name: str) -> _Site:
        s = self.sites.get(name)
        if s is None:
            if len(self.sites) >= self.max_sites:
                raise ProcessingError.limit_exceeded("tensor-parallel call sites", self.max_sites,
                                                     len(self.sites) + 1)
            s = _Site()
            s.index = len(self.sites)
            self.sites[name] = s
        return s

    def gather_buffer(self, name: str, T: int, K: int) -> torch.Tensor:
        """The symmetric ``[T, K]`` bf16 buffer of an all-gather site.  The caller writes rows
        ``[rank*T/tp, (rank+1)*T/tp)`` (see :meth:`own_rows`) and then calls :meth:`ag_gemm`."""
        s = self._site(name)
        if getattr(s, "shape", None) != (T, K):
            s.shape = (T, K)
            if self.backend == "fused":
                from .symm import SymmetricBuffer
                s.sym = SymmetricBuffer(T * K * 2, self.group, self.device)
                s.buf = s.sym.view(torch.bfloat16, 0, T * K).view(T, K)
                s.flags = torch.zeros((T + 127) // 128, dtype=torch.int32, device=self.device)
            else:
                s.buf = torch.empty((T, K), dtype=torch.bfloat16 if self.device.type == "cuda"
                                    else torch.float32, device=self.device)
        return s.buf

    def own_rows(self, name: str, T: int, K: int) -> torch.Tensor:
        """View of this rank's rows of the gather buffer; waits (on the stream) until every peer
        has finished pulling the previous contents."""
        buf = self.gather_buffer(name, T, K)
        s = self.sites[name]
        if self.backend == "fused" and s.epoch > 0:
            self.pad.wait(2 * s.index + 1, s.epoch)
        Ts = T // self.tp
        return buf[self.rank * Ts:(self.rank + 1) * Ts]

    # ------------------------------------------------------------------ all-gather -> GEMM
    def ag_gemm(self, name: str, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, b_mn: bool = True
                ) -> Tuple[torch.Tensor, torch.Tensor]:
        """``y[T, N] = gather(x)[T, K] @ w (+ bias)`` for the site's gather buffer whose own rows
        were just written; ``w`` is ``[K, N]`` (``b_mn=True``) or ``[N, K]`` (``b_mn=False``, the
        transposed use in the backward pass).  Returns ``(y, gathered x)``."""
        s = self.sites[name]
        T, K = s.shape
        Ts = T // self.tp
        N = w.shape[1] if b_mn else w.shape[0]
        x = s.buf
        s.epoch += 1
        if self.backend == "nccl" or self.tp == 1:
            if self.tp > 1:
                own = x[self.rank * Ts:(self.rank + 1) * Ts].contiguous()
                dist.all_gather_into_tensor(x, own, group=self.group)
            y = G.gemm(x, w, b_mn=b_mn, bias=bias, out=out)
            return y, x
        if Ts % 128 != 0:
            raise ProcessingError.invalid_input(
                f"fused all-gather GEMM needs rows per rank ({Ts}) to be a multiple of 128")
        if out is None:
            out = torch.empty((T, N), dtype=torch.bfloat16, device=self.device)
        self.pad.signal(2 * s.index, s.epoch)
        c = _CommArgs()
        c.comm, c.tp, c.rank, c.rows_per_shard = 1, self.tp, self.rank, Ts
        for r in range(self.tp):
            c.ag_src[r] = s.sym.ptrs[r]
        c.ag_flags = s.flags.data_ptr()
        c.ag_epoch = s.epoch
        c.peer_flags = self.pad.buf.local_ptr + 8 * (2 * s.index) * self.tp
        c.peer_expect = s.epoch
        c.wait_limit_ns = self.limit_ns
        st = _lib.status_buffer(self.device)
        rc = _lib.lib().cb_gemm_bf16_fused(
            _lib.ptr(x), _lib.ptr(w), _lib.ptr(out), T, N, K, x.stride(0), w.stride(0),
            out.stride(0), int(b_mn), _lib.ptr(bias), 256 if N > 128 else 128, ctypes.byref(c),
            _lib.ptr(st), 0, _lib.stream_ptr())
        _lib.check_rc(rc, "cb_gemm_bf16_fused(ag)")
        self.pad.signal(2 * s.index + 1, s.epoch)   # "I have pulled your rows"
        return out, x

    # ------------------------------------------------------------------ GEMM -> reduce-scatter
    def gemm_rs(self, name: str, a: torch.Tensor, w: torch.Tensor,
                resid: Optional[torch.Tensor] = None, b_mn: bool = True) -> torch.Tensor:
        """``out[T/tp, N] = reduce_scatter_rows(a[T, K_local] @ w) (+ resid)``.  ``w`` is
        ``[K_local, N]`` (``b_mn=True``) or ``[N, K_local]`` (``b_mn=False``, the transposed use
        in the backward pass)."""
        s = self._site(name)
        T = a.shape[0]
        Ts = T // self.tp
        N = w.shape[1] if b_mn else w.shape[0]
        s.epoch += 1
        if self.backend == "nccl" or self.tp == 1:
            full = G.gemm(a, w, b_mn=b_mn)
            if self.tp == 1:
                return full if resid is None else (full.float() + resid.float()).to(full.dtype)
            out = torch.empty((Ts, N), dtype=full.dtype, device=full.device)
            if full.is_cuda:
                dist.reduce_scatter_tensor(out, full, group=self.group)
            else:
                dist.all_reduce(full, group=self.group)
                out.copy_(full[self.rank * Ts:(self.rank + 1) * Ts])
            if resid is not None:
                out = (out.float() + resid.float()).to(out.dtype)
            return out
        if Ts % 128 != 0:
            raise ProcessingError.invalid_input(
                f"fused GEMM reduce-scatter needs rows per rank ({Ts}) to be a multiple of 128")
        if getattr(s, "shape", None) != (Ts, N):
            from .symm import SymmetricBuffer
            s.shape = (Ts, N)
            s.sym = SymmetricBuffer(self.tp * Ts * N * 2, self.group, self.device)
            s.slots = s.sym.view(torch.bfloat16, 0, self.tp * Ts * N).view(self.tp, Ts, N)
        if s.epoch > 1:   # every owner must have consumed what we pushed last time
            self.pad.wait(2 * s.index + 1, s.epoch - 1)
        K = a.shape[1]
        c = _CommArgs()
        c.comm, c.tp, c.rank, c.rows_per_shard = 2, self.tp, self.rank, Ts
        for r in range(self.tp):
            c.rs_dst[r] = s.sym.ptrs[r] + self.rank * Ts * N * 2
        c.rs_ld = N
        c.wait_limit_ns = self.limit_ns
        st = _lib.status_buffer(self.device)
        rc = _lib.lib().cb_gemm_bf16_fused(
            _lib.ptr(a), _lib.ptr(w), _lib.ptr(None), T, N, K, a.stride(0), w.stride(0), N,
            int(b_mn), _lib.ptr(None), 256 if N > 128 else 128, ctypes.byref(c), _lib.ptr(st), 0,
            _lib.stream_ptr())
        _lib.check_rc(rc, "cb_gemm_bf16_fused(rs)")
        self.pad.signal(2 * s.index, s.epoch)            # "my partial rows are in your slot"
        self.pad.wait(2 * s.index, s.epoch)              # all peers' rows are in mine
        out = torch.empty((Ts, N), dtype=torch.bfloat16, device=self.device)
        rc = _lib.lib().cb_reduce_slots(_lib.ptr(s.slots), self.tp, Ts, N, N, _lib.ptr(resid),
                                        resid.stride(0) if resid is not None else 0,
                                        _lib.ptr(out), out.stride(0), _lib.stream_ptr())
        _lib.check_rc(rc, "cb_reduce_slots")
        self.pad.signal(2 * s.index + 1, s.epoch)        # "slots consumed"
        return out

    # ------------------------------------------------------------------ small collectives
    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        if self.tp > 1:
            dist.all_reduce(t, group=self.group)
        return t
