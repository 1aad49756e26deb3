"""Context parallelism (ring attention): one sequence is split over the ranks of a group, every
rank keeps the queries of its own tokens and visits the keys/values of all ranks.

Layout.  A sequence of ``S`` tokens is cut into ``2 * cp`` chunks of ``Sc`` tokens; rank ``r`` owns
chunks ``r`` and ``2 * cp - 1 - r`` (zig-zag), which gives every rank the same amount of causal
work: against each other rank exactly two full (unmasked) chunk pairs.  Local activations are
chunk-major, ``[2, B, Sc, ...]`` flattened to rows, so a chunk is a contiguous ``[B * Sc, H]`` block
that the attention kernels take as ``B`` sequences of length ``Sc``.

Forward.  For each source rank the (query chunk, key/value chunk) pairs that are not fully masked
run through the single-GPU flash-attention kernel; the partial ``(O, lse)`` results are folded into
an fp32 running result (``csrc/ring.cu: attn_merge``).  Backward re-visits the same pairs with the
final ``lse`` and output, accumulates ``dQ`` locally and sends each ``dK/dV`` contribution home.

Transport.  ``backend="p2p"``: each rank publishes its K/V in a symmetric buffer; a side stream
pulls the peers' buffers over NVLink into local staging buffers while the main stream is already
computing on what has arrived (the attention kernel then TMA-loads local memory only); key/value
gradients are reduced straight into the owner's fp32 buffer with system-scope ``red.add``.
``backend="collective"``: all-gather of K/V and all-reduce / reduce-scatter of the gradients (the
baseline, and the path of CPU ranks).  The reference bounds the context by ``max_seq_len`` and
materialises S x S scores per head (plugins/model-transformer/src/lib.rs:237-277,797-802).
"""
from __future__ import annotations

from typing import Iterator, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..foundation.error import ProcessingError
from ..ops import attention as A
from ..ops import ring as R


class ContextParallel:
    n_chunks = 2     # sequence chunks a rank owns (leading dimension of the ids it is given)

    def __init__(self, group, device, backend: Optional[str] = None,
                 wait_limit_ms: float = 5000.0) -> None:
        self.group = group
        self.device = torch.device(device)
        self.rank = dist.get_rank(group) if group is not None else 0
        self.cp = dist.get_world_size(group) if group is not None else 1
        if backend is None:
            backend = "p2p" if self.device.type == "cuda" and self.cp > 1 else "collective"
        self.backend = backend
        self.limit_ms = wait_limit_ms
        self.pad = None
        self._kv_sym = self._dkv_sym = None
        self._kv_epoch = self._dkv_epoch = 0
        self._staging: List[torch.Tensor] = []
        self._side = None
        if backend == "p2p":
            from .symm import SignalPad
            self.pad = SignalPad(4, group, self.device, wait_limit_ms)
            self._side = torch.cuda.Stream(self.device)

    # ------------------------------------------------------------------ layout
    @property
    def chunk_ids(self) -> Tuple[int, int]:
        return self.rank, 2 * self.cp - 1 - self.rank

    def shard(self, x: torch.Tensor) -> torch.Tensor:
        """``[B, S, ...] -> [2, B, Sc, ...]``: this rank's two chunks of every sequence."""
        B, S = x.shape[0], x.shape[1]
        if S % (2 * self.cp):
            raise ProcessingError.invalid_input(
                f"sequence length {S} is not a multiple of 2 * cp = {2 * self.cp}")
        Sc = S // (2 * self.cp)
        c = x.reshape(B, 2 * self.cp, Sc, *x.shape[2:])
        a, b = self.chunk_ids
        return torch.stack([c[:, a], c[:, b]], 0).contiguous()

    def position_offsets(self, Sc: int) -> Tuple[int, int]:
        a, b = self.chunk_ids
        return a * Sc, b * Sc

    def _pairs(self, src: int) -> List[Tuple[int, int, bool]]:
        """``(query chunk slot, key chunk slot, causal)`` of everything not fully masked."""
        out = []
        kv_ids = (src, 2 * self.cp - 1 - src)
        for qi, a in enumerate(self.chunk_ids):
            for kj, b in enumerate(kv_ids):
                if b < a:
                    out.append((qi, kj, False))
                elif b == a:
                    out.append((qi, kj, True))
        return out

    # ------------------------------------------------------------------ key/value transport
    def _sources(self, kv: torch.Tensor) -> Iterator[Tuple[int, torch.Tensor]]:
        """Yields ``(source rank, its [2*Tc, 2H] keys|values)``, own first, then ring order."""
        r, cp = self.rank, self.cp
        if cp == 1:
            yield 0, kv
            return
        if self.backend != "p2p":
            mine = kv.contiguous()
            parts = [torch.empty_like(mine) for _ in range(cp)]
            dist.all_gather(parts, mine, group=self.group)
            yield r, mine
            for t in range(1, cp):
                yield (r - t) % cp, parts[(r - t) % cp]
            return
        from .symm import SymmetricBuffer
        from ..ops import _lib
        import ctypes
        nbytes = kv.numel() * 2
        if self._kv_sym is None or self._kv_sym.nbytes < nbytes:
            self._kv_sym = SymmetricBuffer(nbytes, self.group, self.device)
            self._staging = []
            self._kv_epoch = 0
        sym = self._kv_sym
        if self._kv_epoch > 0:
            self.pad.wait(1, self._kv_epoch)          # every peer has pulled what I published last
        self._kv_epoch += 1
        epoch = self._kv_epoch
        local = sym.view(torch.bfloat16, 0, kv.numel()).view(kv.shape)
        local.copy_(kv)
        self.pad.signal(0, epoch)
        while len(self._staging) < cp - 1 or self._staging[0].shape != kv.shape:
            if self._staging and self._staging[0].shape != kv.shape:
                self._staging = []
            self._staging.append(torch.empty(kv.shape, dtype=torch.bfloat16, device=self.device))
        main = torch.cuda.current_stream()
        self._side.wait_stream(main)                   # staging buffers are free again
        events = []
        with torch.cuda.stream(self._side):
            self.pad.wait(0, epoch)                    # all peers have published
            for t in range(1, cp):
                s = (r - t) % cp
                rc = _lib.lib().cb_peer_copy(ctypes.c_void_p(sym.ptrs[s]),
                                             _lib.ptr(self._staging[t - 1]),
                                             ctypes.c_size_t(nbytes), 0, _lib.stream_ptr())
                _lib.check_rc(rc, "cb_peer_copy")
                ev = torch.cuda.Event()
                ev.record(self._side)
                events.append(ev)
            self.pad.signal(1, epoch)                  # my pulls are done
        yield r, local
        for t in range(1, cp):
            main.wait_event(events[t - 1])
            yield (r - t) % cp, self._staging[t - 1]

    # ------------------------------------------------------------------ forward
    def attention_fwd(self, qkv: torch.Tensor, B: int, Sc: int, nh: int, dh: int
                      ) -> Tuple[torch.Tensor, torch.Tensor]:
        """``qkv [2*B*Sc, 3H]`` chunk-major -> ``(o [2*B*Sc, H], lse [2, B, nh, Sc])``."""
        H, Tc = nh * dh, B * Sc
        o_acc = torch.empty((2 * Tc, H), dtype=torch.float32, device=qkv.device)
        lse = torch.empty((2, B, nh, Sc), dtype=torch.float32, device=qkv.device)
        started = [False, False]
        for s, kv in self._sources(qkv[:, H:3 * H]):
            for qi, kj, causal in self._pairs(s):
                q = qkv[qi * Tc:(qi + 1) * Tc, :H]
                k = kv[kj * Tc:(kj + 1) * Tc, :H]
                v = kv[kj * Tc:(kj + 1) * Tc, H:2 * H]
                o_p, lse_p = A.attention_fwd(q, k, v, B, Sc, nh, dh, causal=causal)
                R.merge_partial(o_acc[qi * Tc:(qi + 1) * Tc], lse[qi], o_p, lse_p, B, Sc, nh, dh,
                                first=not started[qi])
                started[qi] = True
        o = torch.empty((2 * Tc, H), dtype=qkv.dtype, device=qkv.device)
        R.cast_rows(o_acc, o)
        return o, lse

    # ------------------------------------------------------------------ backward
    def attention_bwd(self, do: torch.Tensor, qkv: torch.Tensor, o: torch.Tensor,
                      lse: torch.Tensor, B: int, Sc: int, nh: int, dh: int,
                      dqkv: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Gradient ``[2*B*Sc, 3H]`` of the chunk-major fused projection output."""
        H, Tc = nh * dh, B * Sc
        r, cp = self.rank, self.cp
        dev = qkv.device
        dq_acc = torch.zeros((2 * Tc, H), dtype=torch.float32, device=dev)
        p2p = self.backend == "p2p" and cp > 1
        if p2p:
            from .symm import SymmetricBuffer
            nbytes = 2 * Tc * 2 * H * 4
            if self._dkv_sym is None or self._dkv_sym.nbytes < nbytes:
                self._dkv_sym = SymmetricBuffer(nbytes, self.group, self.device)
                self._dkv_epoch = 0
            home = self._dkv_sym.view(torch.float32, 0, 2 * Tc * 2 * H).view(2 * Tc, 2 * H)
            home.zero_()
            self._dkv_epoch += 1
            self.pad.signal(2, self._dkv_epoch)        # my accumulator is cleared
            self.pad.wait(2, self._dkv_epoch)          # ... and so is everyone's
        else:
            full = torch.zeros((cp, 2 * Tc, 2 * H), dtype=torch.float32, device=dev)
        for s, kv in self._sources(qkv[:, H:3 * H]):
            part = torch.zeros((2 * Tc, 2 * H), dtype=torch.float32, device=dev) if p2p else full[s]
            for qi, kj, causal in self._pairs(s):
                rows_q = slice(qi * Tc, (qi + 1) * Tc)
                rows_k = slice(kj * Tc, (kj + 1) * Tc)
                dq, dk, dv = A.attention_bwd(do[rows_q], qkv[rows_q, :H], kv[rows_k, :H],
                                             kv[rows_k, H:2 * H], o[rows_q], lse[qi], B, Sc, nh,
                                             dh, causal=causal)
                R.accum_rows(dq_acc[rows_q], dq)
                R.accum_rows(part[rows_k, :H], dk)
                R.accum_rows(part[rows_k, H:], dv)
            if p2p:
                R.peer_add_f32(self._dkv_sym.ptrs[s], part)
        if p2p:
            self.pad.signal(3, self._dkv_epoch)        # my contributions have landed
            self.pad.wait(3, self._dkv_epoch)          # ... and so have everyone's
            dkv = home
        elif cp > 1:
            if dev.type == "cuda":
                dkv = torch.empty((2 * Tc, 2 * H), dtype=torch.float32, device=dev)
                dist.reduce_scatter_tensor(dkv, full, group=self.group)
            else:
                dist.all_reduce(full, group=self.group)
                dkv = full[r]
        else:
            dkv = full[0]
        if dqkv is None:
            dqkv = torch.empty((2 * Tc, 3 * H), dtype=qkv.dtype, device=dev)
        R.cast_rows(dq_acc, dqkv[:, :H])
        R.cast_rows(dkv, dqkv[:, H:3 * H])
        return dqkv
