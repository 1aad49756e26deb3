"""Tensor-parallel generation engine: weights and KV cache sharded by heads / columns over the
group (the sharding of :class:`coeus_b200.parallel.tp_model.TPDecoderLM`), every rank fed the same
requests.

Prefill runs the sequence-parallel layer (all-gather->GEMM, GEMM->reduce-scatter fused kernels)
over all prompt tokens and writes each rank's heads into its paged cache.  Decode keeps the
``[B, H]`` activations replicated: per layer two GEMMs produce partial sums that the one-shot
all-reduce kernel sums over NVLink together with the residual add and the next norm.  A decode
step has no host-dependent launch parameter (positions live on the device), so it is captured
once in a CUDA graph and replayed.  Greedy selection exchanges one (value, index) pair per
sequence and rank instead of the logits.  The reference generates by re-running its whole
forward per token on one CPU thread (src/core/model.rs:138-144 names ``generate`` only)."""
from __future__ import annotations

import time
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..foundation.error import ProcessingError
from ..ops import attention as A
from ..ops import decode as D
from ..ops import elementwise as E
from ..ops import gemm as G
from ..ops import norm as N
from ..parallel.allreduce import FusedAllReduce
from ..parallel.tp_model import TPDecoderLM
from .kv_cache import PagedKVCache


class TPInferenceEngine:
    def __init__(self, model: TPDecoderLM, max_batch: int = 64, use_graph: Optional[bool] = None,
                 ar_backend: Optional[str] = None, decode_splits: int = 0) -> None:
        self.m, self.cfg, self.tp = model, model.cfg, model.tp
        self.device = model.device
        self.max_batch = max_batch
        self.max_len = self.cfg.max_seq_len
        self.decode_splits = decode_splits
        cuda = self.device.type == "cuda"
        self.use_graph = (cuda and self.cfg.pos != "sinusoidal") if use_graph is None else use_graph
        self.ar = FusedAllReduce(self.tp.group, self.device, max_batch, self.cfg.hidden_dim,
                                 backend=ar_backend, dtype=model.p16.dtype)
        self._select = None
        if self.ar.backend in ("fused", "nvls"):
            from ..parallel.allreduce import GreedySelect
            self._select = GreedySelect(self.tp.group, self.device, max_batch)
        self.cache: Optional[PagedKVCache] = None
        # positions live in buffers that are never reallocated: a captured graph reads them
        self._pos_buf = torch.zeros(max_batch, dtype=torch.int32, device=self.device)
        self._ctx_buf = torch.zeros(max_batch, dtype=torch.int32, device=self.device)
        self._graph = None
        self._graph_B = 0
        self.stats: Dict[str, float] = {}

    # ------------------------------------------------------------------ helpers
    def _ensure_cache(self, B: int, total: int) -> PagedKVCache:
        c = self.cache
        need_pages = (total + D.PAGE - 1) // D.PAGE
        if c is None or c.page_table.shape[0] < B or c.page_table.shape[1] < need_pages:
            c = PagedKVCache.for_model(self.cfg, max(B, 1), max(total, D.PAGE), self.device,
                                       heads=self.m.kvh_l)
            if self.m.p16.dtype != torch.bfloat16:
                c.k = [t.to(self.m.p16.dtype) for t in c.k]
                c.v = [t.to(self.m.p16.dtype) for t in c.v]
            self.cache = c
            self._graph = None
        for b in list(c.owned):
            c.release(b)
        for b in range(B):
            c.reserve(b, total)
        return c

    def _norm(self, x, prefix):
        m = self.m
        y, _, _ = N.norm_fwd(x, m.w[prefix + "_scale"], None if m.rms else m.w[prefix + "_bias"],
                             self.cfg.norm_eps, m.rms)
        return y

    def _norm_params(self, prefix):
        m = self.m
        return m.w[prefix + "_scale"], (None if m.rms else m.w[prefix + "_bias"])

    # ------------------------------------------------------------------ prefill
    def prefill(self, ids: torch.Tensor, total_len: int) -> torch.Tensor:
        """Prompt ``ids [B, S]`` (the same on every rank) -> this rank's slice ``[B, V/tp]`` of the
        last position's logits; fills the cache."""
        m, cfg, tp = self.m, self.cfg, self.tp
        B, S = ids.shape
        T, n, r = B * S, m.n, m.rank
        if T % n:
            raise ProcessingError.invalid_input(f"B*S = {T} must be divisible by tp = {n}")
        Ts = T // n
        if Ts % S and S % Ts:
            raise ProcessingError.invalid_input("tokens per rank must divide or be a multiple of S")
        cache = self._ensure_cache(B, total_len)
        H, dh, nh, Hl = cfg.hidden_dim, cfg.head_dim, m.nh_l, m.Hl
        my_ids = ids.reshape(-1)[r * Ts:(r + 1) * Ts].contiguous()
        pos_off = (r * Ts) % S if Ts < S else 0
        x = E.embed_fwd(my_ids, m.w["token_embed"], m._positions(max(S, total_len)), S,
                        pos_offset=pos_off)
        pos0 = torch.zeros(B, dtype=torch.int32, device=self.device)
        for l in range(cfg.num_layers):
            p = f"layers.{l}."
            tp.own_rows("ag_attn", T, H).copy_(self._norm(x, p + "norm1"))
            qkv, _ = tp.ag_gemm("ag_attn", m.w[p + "attn.qkv_weights"])
            if cfg.pos == "rope":
                m._rope(qkv, S)
            q, k, v = m._split_qkv(qkv, expand=False)   # the cache keeps the rank's K/V heads
            D.kv_write(k, v, cache.k[l], cache.v[l], cache.page_table, pos0, S, m.kvh_l, dh)
            attn, _ = A.attention_fwd(q, k, v, B, S, nh, dh, causal=True)
            x_mid = tp.gemm_rs("rs_attn", attn, m.w[p + "attn.o_weights"], resid=x)
            tp.own_rows("ag_mlp", T, H).copy_(self._norm(x_mid, p + "norm2"))
            u, _ = tp.ag_gemm("ag_mlp", m.w[p + "ff.up_weights"])
            act = E.swiglu_fwd(u) if m.swiglu else E.gelu_fwd(u)
            x = tp.gemm_rs("rs_mlp", act, m.w[p + "ff.down_weights"], resid=x_mid)
        # last position of every sequence: owned by one rank each, summed into a replicated [B, H]
        last = torch.zeros((B, H), dtype=x.dtype, device=self.device)
        t_last = torch.arange(B, device=self.device) * S + (S - 1)
        mine = (t_last >= r * Ts) & (t_last < (r + 1) * Ts)
        if bool(mine.any()):
            last[mine] = x[(t_last[mine] - r * Ts)]
        if n > 1:
            dist.all_reduce(last, group=tp.group)
        if B > self.max_batch:
            raise ProcessingError.limit_exceeded("batch size", self.max_batch, B)
        self._pos0, self._ctx = self._pos_buf[:B], self._ctx_buf[:B]
        self._pos0.fill_(S)
        self._ctx.fill_(S)
        self._pos_host = S
        xf = self._norm(last, "final_norm")
        return G.gemm(xf, m.w["output_proj"], b_mn=True)

    # ------------------------------------------------------------------ slot-wise API (serving)
    def open_slots(self, max_seqs: int, max_len: int) -> PagedKVCache:
        """A cache whose rows are independent request slots (this rank's heads of each)."""
        c = PagedKVCache.for_model(self.cfg, max_seqs, max(max_len, D.PAGE), self.device,
                                   heads=self.m.kvh_l)
        if self.m.p16.dtype != torch.bfloat16:
            c.k = [t.to(self.m.p16.dtype) for t in c.k]
            c.v = [t.to(self.m.p16.dtype) for t in c.v]
        self.cache, self._graph = c, None
        return c

    def _replicated_layers(self, x: torch.Tensor, n_seq: int, S: int, pos0: torch.Tensor,
                           pos_host: int, table: torch.Tensor, ctx: Optional[torch.Tensor],
                           pos_dev: Optional[torch.Tensor]) -> torch.Tensor:
        """All layers on replicated activations ``[n_seq * S, H]``: column-parallel GEMMs give
        this rank's heads / FFN columns, row-parallel GEMMs give partial sums that are added over
        the group.  Prompts of any length go through here (``ctx is None``: causal attention over
        the ``S`` new tokens; else one token per sequence against the paged cache).  Rows beyond
        what the fused all-reduce buffers hold are summed with the library collective."""
        m, cfg, ar, cache = self.m, self.cfg, self.ar, self.cache
        dh, nh, Hl = cfg.head_dim, m.nh_l, m.Hl
        T = x.shape[0]
        fused = T <= self.max_batch

        def reduce(partial_of, resid, norm_prefix):
            if fused:
                partial_of(ar.next_part(T))
                return ar.reduce(T, resid, *self._norm_params(norm_prefix), m.rms, cfg.norm_eps)
            part = torch.empty((T, cfg.hidden_dim), dtype=x.dtype, device=self.device)
            partial_of(part)
            if m.n > 1:
                dist.all_reduce(part, group=self.tp.group)
            y = (part.float() + resid.float()).to(x.dtype)
            return y, self._norm(y, norm_prefix)

        n1 = self._norm(x, "layers.0.norm1")
        L = cfg.num_layers
        for l in range(L):
            p = f"layers.{l}."
            qkv = G.gemm(n1, m.w[p + "attn.qkv_weights"], b_mn=True)
            if cfg.pos == "rope":
                m._rope(qkv, S, pos_offset=pos_host, pos_dev=pos_dev)
            q, k, v = m._split_qkv(qkv, expand=False)   # the cache keeps the rank's K/V heads
            D.kv_write(k, v, cache.k[l], cache.v[l], table, pos0, S, m.kvh_l, dh)
            if ctx is None:
                attn, _ = A.attention_fwd(q, k, v, n_seq, S, nh, dh, causal=True)
            else:
                attn = D.decode_attention(q, cache.k[l], cache.v[l], table, ctx, nh, dh,
                                          splits=self.decode_splits, nkv=m.kvh_l)
            x, n2 = reduce(lambda out: G.gemm(attn, m.w[p + "attn.o_weights"], b_mn=True, out=out),
                           x, p + "norm2")
            u = G.gemm(n2, m.w[p + "ff.up_weights"], b_mn=True)
            act = E.swiglu_fwd(u) if m.swiglu else E.gelu_fwd(u)
            nxt = f"layers.{l + 1}.norm1" if l + 1 < L else "final_norm"
            x, n1 = reduce(lambda out: G.gemm(act, m.w[p + "ff.down_weights"], b_mn=True, out=out),
                           x, nxt)
        return n1            # final-norm output

    def _full_logits(self, xf: torch.Tensor) -> torch.Tensor:
        """``[T, V]`` logits on every rank from the vocabulary-parallel head."""
        m = self.m
        loc = G.gemm(xf, m.w["output_proj"], b_mn=True)            # [T, V/tp]
        if m.n == 1:
            return loc[:, :self.cfg.vocab_size]
        parts = [torch.empty_like(loc) for _ in range(m.n)]
        dist.all_gather(parts, loc.contiguous(), group=self.tp.group)
        return torch.cat(parts, 1)[:, :self.cfg.vocab_size]

    def prefill_slot(self, slot: int, ids: torch.Tensor, total_len: int,
                     token_chunk: Optional[int] = None) -> torch.Tensor:
        """Prompt ``ids [S]`` (any length, the same on every rank) into cache row ``slot``;
        returns the last position's logits ``[V]``.  ``token_chunk`` is accepted for interface
        parity with the single-GPU engine and ignored (the prompt runs in one pass)."""
        m, cfg, cache = self.m, self.cfg, self.cache
        S = ids.numel()
        cache.reserve(slot, total_len)
        x = E.embed_fwd(ids.reshape(-1), m.w["token_embed"], m._positions(max(S, total_len)), S)
        pos0 = torch.zeros(1, dtype=torch.int32, device=self.device)
        xf = self._replicated_layers(x, 1, S, pos0, 0, cache.page_table[slot:slot + 1], None, None)
        cache.set_length(slot, S)
        return self._full_logits(xf[-1:].contiguous())[0]

    def decode_slots(self, slots: torch.Tensor, tokens: torch.Tensor,
                     positions: torch.Tensor) -> torch.Tensor:
        """One token for each cache row in ``slots [n]`` at ``positions [n]`` (int32); returns the
        full ``[n, V]`` logits on every rank."""
        m, cfg, cache = self.m, self.cfg, self.cache
        x = E.embed_fwd(tokens, m.w["token_embed"], None, 1)
        if cfg.pos == "sinusoidal":
            pe = m._positions(int(positions.max()) + 1)
            x = (x.float() + pe[positions.long()].float()).to(x.dtype)
        table = cache.page_table.index_select(0, slots)
        ctx = (positions + 1).to(torch.int32)
        xf = self._replicated_layers(x, tokens.shape[0], 1, positions, 0, table, ctx,
                                     positions if cfg.pos == "rope" else None)
        return self._full_logits(xf)

    # ------------------------------------------------------------------ decode
    def _decode_body(self, tokens: torch.Tensor) -> torch.Tensor:
        """One token per sequence at position ``_pos0`` -> local logits ``[B, V/tp]``; advances
        the device-side positions."""
        m, cfg, ar = self.m, self.cfg, self.ar
        B = tokens.shape[0]
        dh, nh, Hl = cfg.head_dim, m.nh_l, m.Hl
        cache = self.cache
        if cfg.pos == "sinusoidal":
            x = E.embed_fwd(tokens, m.w["token_embed"], m._positions(self._pos_host + 1), 1,
                            pos_offset=self._pos_host)
        else:
            x = E.embed_fwd(tokens, m.w["token_embed"], None, 1)
        self._ctx.add_(1)
        n1 = self._norm(x, "layers.0.norm1")
        L = cfg.num_layers
        for l in range(L):
            p = f"layers.{l}."
            qkv = G.gemm(n1, m.w[p + "attn.qkv_weights"], b_mn=True)
            if cfg.pos == "rope":
                m._rope(qkv, 1, pos_dev=self._pos0)
            q, k, v = m._split_qkv(qkv, expand=False)   # the cache keeps the rank's K/V heads
            D.kv_write(k, v, cache.k[l], cache.v[l], cache.page_table, self._pos0, 1, m.kvh_l, dh)
            attn = D.decode_attention(q, cache.k[l], cache.v[l], cache.page_table, self._ctx, nh,
                                      dh, splits=self.decode_splits, nkv=m.kvh_l)
            G.gemm(attn, m.w[p + "attn.o_weights"], b_mn=True, out=ar.next_part(B))
            x, n2 = ar.reduce(B, x, *self._norm_params(p + "norm2"), m.rms, cfg.norm_eps)
            u = G.gemm(n2, m.w[p + "ff.up_weights"], b_mn=True)
            act = E.swiglu_fwd(u) if m.swiglu else E.gelu_fwd(u)
            G.gemm(act, m.w[p + "ff.down_weights"], b_mn=True, out=ar.next_part(B))
            nxt = f"layers.{l + 1}.norm1" if l + 1 < L else "final_norm"
            x, n1 = ar.reduce(B, x, *self._norm_params(nxt), m.rms, cfg.norm_eps)
        self._pos0.add_(1)
        return G.gemm(n1, m.w["output_proj"], b_mn=True)

    def _greedy_from_local(self, logits_l: torch.Tensor) -> torch.Tensor:
        """Arg-max over the whole vocabulary from each rank's ``[B, V/tp]`` slice."""
        m = self.m
        B = logits_l.shape[0]
        V, Vl = self.cfg.vocab_size, m.Vl
        valid = min(Vl, max(0, V - m.rank * Vl))        # padding columns do not compete
        if self._select is not None and (self._select._batch in (None, B)):
            return self._select.select(logits_l, valid, m.rank * Vl)
        idx = D.argmax_rows(logits_l[:, :valid]) if valid > 0 else \
            torch.zeros(B, dtype=torch.int64, device=logits_l.device)
        val = logits_l.float().gather(1, idx[:, None])[:, 0] if valid > 0 else \
            torch.full((B,), float("-inf"), device=logits_l.device)
        if m.n == 1:
            return idx
        pair = torch.stack([val, (idx + m.rank * Vl).float()], 1).contiguous()   # ids < 2^24
        flat = torch.empty((m.n * B, 2), dtype=torch.float32, device=logits_l.device)
        dist.all_gather_into_tensor(flat, pair, group=self.tp.group)
        allp = flat.view(m.n, B, 2)
        best = allp[:, :, 0].argmax(0)                   # first rank wins ties, as one arg-max would
        return allp[best, torch.arange(B, device=best.device), 1].long()

    def decode_step(self, tokens: torch.Tensor, greedy: bool = True) -> torch.Tensor:
        """``tokens [B]`` -> next tokens ``[B]`` (greedy) or this rank's logits slice."""
        B = tokens.shape[0]
        if not self.use_graph:
            out = self._decode_body(tokens)
            self._pos_host += 1
            return self._greedy_from_local(out) if greedy else out
        if self._graph is None or self._graph_B != B or self._graph_greedy != greedy:
            self._tok_in = tokens.clone()
            keep = (self._pos0.clone(), self._ctx.clone(), self.ar._turn)
            side = torch.cuda.Stream(self.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):               # warm-up outside the capture
                self._decode_body(self._tok_in)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.tp.group) if self.m.n > 1 else None
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph):
                out = self._decode_body(self._tok_in)
                self._graph_out = self._greedy_from_local(out) if greedy else out
            # warm-up and capture each advanced the positions and wrote one cache slot: rewind
            self._pos0.copy_(keep[0])
            self._ctx.copy_(keep[1])
            self._graph_B, self._graph_greedy = B, greedy
        self._tok_in.copy_(tokens)
        self._graph.replay()
        self._pos_host += 1
        return self._graph_out.clone()

    def close(self) -> None:
        """Drop the captured graph (before the process group is destroyed)."""
        self._graph = None
        self._graph_out = None

    def generate(self, ids: torch.Tensor, max_new_tokens: int) -> torch.Tensor:
        """Greedy generation: ``[B, S] -> [B, S + max_new_tokens]`` (identical on every rank)."""
        B, S = ids.shape
        total = S + max_new_tokens
        out = torch.empty((B, total), dtype=torch.int64, device=ids.device)
        out[:, :S] = ids
        if max_new_tokens == 0:
            return out
        t0 = time.perf_counter()
        nxt = self._greedy_from_local(self.prefill(ids, total))
        if ids.is_cuda:
            torch.cuda.synchronize(ids.device)
        t1 = time.perf_counter()
        out[:, S] = nxt
        for i in range(1, max_new_tokens):
            nxt = self.decode_step(nxt)
            out[:, S + i] = nxt
        if ids.is_cuda:
            torch.cuda.synchronize(ids.device)
        t2 = time.perf_counter()
        self.stats = {"prefill_s": t1 - t0, "decode_s": t2 - t1,
                      "prefill_tokens_per_s": B * S / max(t1 - t0, 1e-9),
                      "decode_tokens_per_s": B * max(0, max_new_tokens - 1) / max(t2 - t1, 1e-9)}
        return out
