"""Generation engine: batched prefill with the flash-attention kernel, then one decode step per
token over a paged KV cache (``csrc/decode_attn.cu``).  Implements what the reference's
``GenerativeModel::generate`` and ``InferenceRequest{tokens, max_length}`` /
``InferenceResult{predictions}`` only name (src/core/model.rs:138-144,
src/domain/inference/mod.rs:6-32); the reference itself recomputes the full sequence for every
token and returns one position."""
from __future__ import annotations

import time
from typing import Dict, List, Optional

import torch

from ..foundation.error import ProcessingError
from ..models.decoder import DecoderLM
from ..ops import attention as A
from ..ops import decode as D
from ..ops import elementwise as E
from ..ops import gemm as G
from ..ops import norm as N
from ..ops import ring as R
from .kv_cache import PagedKVCache
from .sampler import select


class InferenceEngine:
    def __init__(self, model: DecoderLM, max_batch: int = 64, max_len: Optional[int] = None,
                 decode_splits: int = 0, use_graph: Optional[bool] = None) -> None:
        """``use_graph``: capture the decode step in a CUDA graph and replay it per token (default:
        on for CUDA models whose positions are not taken from a host-indexed table).  Positions
        then live in device buffers that are never reallocated."""
        self.m = model
        self.cfg = model.cfg
        self.max_batch = max_batch
        self.max_len = max_len or self.cfg.max_seq_len
        self.decode_splits = decode_splits
        self.cache: Optional[PagedKVCache] = None
        self.stats: Dict[str, float] = {}
        cuda = model.device.type == "cuda"
        self.use_graph = (cuda and self.cfg.pos not in ("sinusoidal", "learned")) \
            if use_graph is None else use_graph
        self._pos_buf = torch.zeros(max_batch, dtype=torch.int32, device=model.device)
        self._ctx_buf = torch.zeros(max_batch, dtype=torch.int32, device=model.device)
        self._graph = None
        self._graph_B = 0

    # ------------------------------------------------------------------ building blocks
    def _ensure_cache(self, B: int, total: int) -> PagedKVCache:
        c = self.cache
        need_pages = (total + D.PAGE - 1) // D.PAGE
        if c is None or c.page_table.shape[0] < B or c.page_table.shape[1] < need_pages:
            c = PagedKVCache.for_model(self.cfg, max(B, 1), max(total, D.PAGE), self.m.device)
            if self.m.p16.dtype != torch.bfloat16:       # CPU oracle runs keep their precision
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
        m, cfg = self.m, self.cfg
        rms = cfg.norm == "rmsnorm"
        y, _, _ = N.norm_fwd(x, m.w[prefix + "_scale"], None if rms else m.w[prefix + "_bias"],
                             cfg.norm_eps, rms)
        return y

    def _mlp(self, p: str, n2: torch.Tensor, resid: torch.Tensor) -> torch.Tensor:
        m, cfg = self.m, self.cfg
        bias = (lambda n: m.w[p + n]) if cfg.use_bias else (lambda n: None)
        if cfg.activation == "swiglu":
            act = E.swiglu_fwd(G.linear_fwd(n2, m.w[p + "ff.gate_up_weights"], None))
            return G.linear_fwd(act, m.w[p + "ff.down_weights"], None, resid=resid)
        act = G.linear_fwd(n2, m.w[p + "ff.up_weights"], bias("ff.up_bias"), epi="gelu")
        return G.linear_fwd(act, m.w[p + "ff.down_weights"], bias("ff.down_bias"), resid=resid)

    def _layers(self, x: torch.Tensor, B: int, S: int, pos0: torch.Tensor, pos0_host: int,
                cache: PagedKVCache, prefill: bool, pos_dev: Optional[torch.Tensor] = None,
                page_table: Optional[torch.Tensor] = None,
                earlier: Optional[List[list]] = None,
                ctx: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``earlier[l]`` (chunked prefill) lists the ``(k, v)`` of the sequence chunks that came
        before this one; this chunk attends to them without a mask, to itself causally, and the
        partial results are merged by their log-sum-exp."""
        m, cfg = self.m, self.cfg
        page_table = cache.page_table if page_table is None else page_table
        H, nh, dh = cfg.hidden_dim, cfg.num_heads, cfg.head_dim
        n1n, n2n, _ = m.layout.norm_names
        for l in range(cfg.num_layers):
            p = f"layers.{l}."
            bias = (lambda n: m.w[p + n]) if cfg.use_bias else (lambda n: None)
            n1 = self._norm(x, p + n1n)
            qkv = G.linear_fwd(n1, m.w[p + "attn.qkv_weights"], bias("attn.qkv_bias"))
            if cfg.pos == "rope" and cfg.rope_llama3 is not None:
                E.rope_freq_(qkv, nh + cfg.kv_heads, dh, S, m.rope_inv_freq(),
                             pos_offset=pos0_host, pos_dev=pos_dev)
            elif cfg.pos == "rope":
                E.rope_(qkv, nh + cfg.kv_heads, dh, S, pos_offset=pos0_host,
                        theta=cfg.rope_theta, pos_dev=pos_dev)
            Hkv = cfg.kv_dim
            q, k, v = qkv[:, :H], qkv[:, H:H + Hkv], qkv[:, H + Hkv:]
            # grouped-query attention: the cache keeps the key/value heads as they are, the
            # prefill and decode kernels index them by query head // group
            D.kv_write(k, v, cache.k[l], cache.v[l], page_table, pos0, S, cfg.kv_heads, dh)
            if prefill:
                attn, lse = A.attention_fwd(q, k, v, B, S, nh, dh, causal=True)
                if earlier is not None:
                    if earlier[l]:
                        acc = torch.empty((B * S, H), dtype=torch.float32, device=x.device)
                        lse_acc = torch.empty_like(lse)
                        R.merge_partial(acc, lse_acc, attn, lse, B, S, nh, dh, True)
                        for kj, vj in earlier[l]:
                            o_p, lse_p = A.attention_fwd(q, kj, vj, B, S, nh, dh, causal=False)
                            R.merge_partial(acc, lse_acc, o_p, lse_p, B, S, nh, dh, False)
                        R.cast_rows(acc, attn)
                    earlier[l].append((k, v))
            else:
                attn = D.decode_attention(q, cache.k[l], cache.v[l], page_table,
                                          self._ctx if ctx is None else ctx, nh, dh,
                                          splits=self.decode_splits, nkv=cfg.kv_heads)
            x_mid = G.linear_fwd(attn, m.w[p + "attn.o_weights"], bias("attn.o_bias"), resid=x)
            x = self._mlp(p, self._norm(x_mid, p + n2n), x_mid)
        return x

    def _logits(self, x_last: torch.Tensor) -> torch.Tensor:
        m = self.m
        xf = self._norm(x_last, m.layout.norm_names[2])
        w, b_mn = m.output_weight()
        return G.gemm(xf, w, b_mn=b_mn)

    # ------------------------------------------------------------------ public API
    def prefill(self, ids: torch.Tensor, total_len: int, seq_chunk: Optional[int] = None,
                token_chunk: Optional[int] = None) -> torch.Tensor:
        """Runs the prompt ``ids [B, S]`` through the model, fills the cache, returns the logits
        of the last position ``[B, V]``.

        Chunking bounds the activation memory of a large prompt batch: ``seq_chunk`` sequences
        are taken at a time, and within them ``token_chunk`` positions at a time (rounded down to
        a divisor of ``S``; every chunk attends to the keys and values of the chunks before it,
        which are kept until the group of sequences is done)."""
        B, S = ids.shape
        if B > self.max_batch:
            raise ProcessingError.limit_exceeded("batch size", self.max_batch, B)
        cache = self._ensure_cache(B, total_len)
        m, cfg = self.m, self.cfg
        nb = B if not seq_chunk else max(1, min(B, int(seq_chunk)))
        Sc = S
        if token_chunk and token_chunk < S:
            Sc = max(d for d in range(1, int(token_chunk) + 1) if S % d == 0)
        pe = m._positions(max(S, total_len))
        last = torch.empty((B, cfg.hidden_dim), dtype=m.p16.dtype, device=m.device)
        for b0 in range(0, B, nb):
            b1 = min(B, b0 + nb)
            Bg = b1 - b0
            table = cache.page_table[b0:b1]
            earlier = [[] for _ in range(cfg.num_layers)] if Sc < S else None
            for c0 in range(0, S, Sc):
                pos0 = torch.full((Bg,), c0, dtype=torch.int32, device=m.device)
                x = E.embed_fwd(ids[b0:b1, c0:c0 + Sc].reshape(-1), m.w["token_embed"], pe, Sc,
                                pos_offset=c0)
                x = self._layers(x, Bg, Sc, pos0, c0, cache, prefill=True, page_table=table,
                                 earlier=earlier)
            last[b0:b1] = x.view(Bg, Sc, -1)[:, -1, :]
        self._pos = S
        self._pos0, self._ctx = self._pos_buf[:B], self._ctx_buf[:B]
        self._pos0.fill_(S)
        self._ctx.fill_(S)
        return self._logits(last)

    # ------------------------------------------------------------------ slot-wise API (serving)
    def open_slots(self, max_seqs: int, max_len: int) -> PagedKVCache:
        """A cache whose rows are independent request slots (see
        :class:`coeus_b200.infer.scheduler.ContinuousBatcher`); pages are handed out per slot."""
        c = PagedKVCache.for_model(self.cfg, max_seqs, max(max_len, D.PAGE) + D.PAGE,
                                   self.m.device)
        if self.m.p16.dtype != torch.bfloat16:       # CPU oracle runs keep their precision
            c.k = [t.to(self.m.p16.dtype) for t in c.k]
            c.v = [t.to(self.m.p16.dtype) for t in c.v]
        self.cache = c
        self._graph = None
        return c

    def prefill_slot(self, slot: int, ids: torch.Tensor, total_len: int,
                     token_chunk: Optional[int] = None) -> torch.Tensor:
        """Prompt ``ids [S]`` of one request into cache row ``slot``; returns its last-position
        logits ``[V]``."""
        cache, m, cfg = self.cache, self.m, self.cfg
        S = ids.numel()
        cache.reserve(slot, total_len)
        Sc = S
        if token_chunk and token_chunk < S:
            Sc = max(d for d in range(1, int(token_chunk) + 1) if S % d == 0)
        pe = m._positions(max(S, total_len))
        table = cache.page_table[slot:slot + 1]
        earlier = [[] for _ in range(cfg.num_layers)] if Sc < S else None
        for c0 in range(0, S, Sc):
            pos0 = torch.full((1,), c0, dtype=torch.int32, device=m.device)
            x = E.embed_fwd(ids[c0:c0 + Sc].reshape(-1), m.w["token_embed"], pe, Sc, pos_offset=c0)
            x = self._layers(x, 1, Sc, pos0, c0, cache, prefill=True, page_table=table,
                             earlier=earlier)
        cache.set_length(slot, S)
        return self._logits(x[-1:].contiguous())[0]

    def prefill_slot_paged(self, slot: int, ids: torch.Tensor, total_len: int,
                           prefix_pages: List[int]) -> torch.Tensor:
        """Like :meth:`prefill_slot`, but the first ``len(prefix_pages) * 64`` prompt tokens are
        not computed: their keys and values already sit in ``prefix_pages`` (filled by an earlier
        request with the same prefix), which the slot adopts.  The rest of the prompt runs in
        page-sized chunks, each attending to the pages before it and causally to itself; the last
        chunk is padded to a full page (rows past the prompt are computed and thrown away, their
        cache entries are overwritten by the decode steps before anything reads them)."""
        cache, m, cfg = self.cache, self.m, self.cfg
        PG = D.PAGE
        S = ids.numel()
        P = len(prefix_pages) * PG
        if not 0 <= P < S:
            raise ProcessingError.invalid_input("the cached prefix must be shorter than the prompt")
        H = cfg.hidden_dim
        cache.adopt(slot, list(prefix_pages))
        padded = P + (S - P + PG - 1) // PG * PG
        cache.reserve(slot, max(total_len, padded))
        pe = m._positions(max(padded, total_len))
        table = cache.page_table[slot:slot + 1]
        Hkv = cfg.kv_dim        # the cache holds the key/value heads
        earlier = [[(cache.k[l][pg].view(PG, Hkv), cache.v[l][pg].view(PG, Hkv))
                    for pg in prefix_pages] for l in range(cfg.num_layers)]
        pad = torch.zeros(padded - S, dtype=ids.dtype, device=ids.device)
        toks = torch.cat([ids, pad])
        for c0 in range(P, padded, PG):
            pos0 = torch.full((1,), c0, dtype=torch.int32, device=m.device)
            x = E.embed_fwd(toks[c0:c0 + PG].reshape(-1), m.w["token_embed"], pe, PG,
                            pos_offset=c0)
            x = self._layers(x, 1, PG, pos0, c0, cache, prefill=True, page_table=table,
                             earlier=earlier)
        cache.set_length(slot, S)
        last = (S - 1) - (padded - PG)
        return self._logits(x[last:last + 1].contiguous())[0]

    def decode_slots(self, slots: torch.Tensor, tokens: torch.Tensor,
                     positions: torch.Tensor) -> torch.Tensor:
        """One token for each of the cache rows ``slots [n]`` (int64): ``tokens [n]`` is fed at
        ``positions [n]`` (int32, the rows' current lengths, which may all differ); returns
        ``[n, V]`` logits.  The caller advances the lengths."""
        cache, m, cfg = self.cache, self.m, self.cfg
        n = tokens.shape[0]
        x = E.embed_fwd(tokens, m.w["token_embed"], None, 1)
        if cfg.pos in ("sinusoidal", "learned"):
            pe = m._positions(int(positions.max()) + 1)
            x = (x.float() + pe[positions.long()].float()).to(x.dtype)
        table = cache.page_table.index_select(0, slots)
        ctx = (positions + 1).to(torch.int32)
        x = self._layers(x, n, 1, positions, 0, cache, prefill=False,
                         pos_dev=positions if cfg.pos == "rope" else None, page_table=table,
                         ctx=ctx)
        return self._logits(x)

    def _decode_body(self, tokens: torch.Tensor) -> torch.Tensor:
        """One token per sequence at the device-side position; advances the positions."""
        m, cfg = self.m, self.cfg
        B = tokens.shape[0]
        pos = self._pos
        if cfg.pos in ("sinusoidal", "learned"):
            x = E.embed_fwd(tokens, m.w["token_embed"], m._positions(pos + 1), 1, pos_offset=pos)
        else:
            x = E.embed_fwd(tokens, m.w["token_embed"], None, 1)
        self._ctx.add_(1)
        x = self._layers(x, B, 1, self._pos0, pos, self.cache, prefill=False,
                         pos_dev=self._pos0 if cfg.pos == "rope" else None)
        self._pos0.add_(1)
        return self._logits(x)

    def decode_step(self, tokens: torch.Tensor) -> torch.Tensor:
        """Feeds one token per sequence (``[B]`` int64) at the next position; returns ``[B, V]``."""
        B = tokens.shape[0]
        if not self.use_graph:
            out = self._decode_body(tokens)
            self._pos += 1
            return out
        if self._graph is None or self._graph_B != B:
            dev = self.m.device
            self._tok_in = tokens.clone()
            keep = (self._pos0.clone(), self._ctx.clone())
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):                # warm-up outside the capture
                self._decode_body(self._tok_in)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize(dev)
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph):
                self._graph_out = self._decode_body(self._tok_in)
            # warm-up and capture advanced the positions and wrote one cache slot: rewind
            self._pos0.copy_(keep[0])
            self._ctx.copy_(keep[1])
            self._graph_B = B
        self._tok_in.copy_(tokens)
        self._graph.replay()
        self._pos += 1
        return self._graph_out

    def generate(self, ids: torch.Tensor, max_new_tokens: int, temperature: float = 0.0,
                 top_k: Optional[int] = None, top_p: Optional[float] = None, seed: int = 0,
                 eos_id: Optional[int] = None, seq_chunk: Optional[int] = None,
                 token_chunk: Optional[int] = None) -> torch.Tensor:
        """Returns ``[B, S + max_new_tokens]`` token ids (prompt included); after ``eos_id`` a
        sequence is padded with ``eos_id`` and decoding stops once all have ended.  ``seq_chunk`` /
        ``token_chunk`` bound the memory of the prompt pass (see :meth:`prefill`)."""
        if ids.dim() == 1:
            ids = ids[None]
        B, S = ids.shape
        total = S + max_new_tokens
        if total > max(self.max_len, self.cfg.max_seq_len) and self.cfg.pos != "rope":
            raise ProcessingError.limit_exceeded("sequence length", self.cfg.max_seq_len, total)
        gen = None
        if temperature and temperature > 0:
            gen = torch.Generator(device=ids.device)
            gen.manual_seed(seed)
        out = torch.empty((B, total), dtype=torch.int64, device=ids.device)
        out[:, :S] = ids
        if max_new_tokens == 0:
            return out
        t0 = time.perf_counter()
        logits = self.prefill(ids, total, seq_chunk=seq_chunk, token_chunk=token_chunk)
        if ids.is_cuda:
            torch.cuda.synchronize(ids.device)
        t1 = time.perf_counter()
        V = self.cfg.vocab_size      # the padding columns of the vocabulary never compete
        nxt = select(logits[:, :V], temperature, top_k, top_p, gen)
        out[:, S] = nxt
        done = (nxt == eos_id) if eos_id is not None else None
        for i in range(1, max_new_tokens):
            if done is not None and bool(done.all()):      # every sequence has ended
                out[:, S + i:] = eos_id
                break
            logits = self.decode_step(nxt)
            nxt = select(logits[:, :V], temperature, top_k, top_p, gen)
            if done is not None:                           # a finished sequence stays finished
                nxt = torch.where(done, torch.full_like(nxt, eos_id), nxt)
                done = done | (nxt == eos_id)
            out[:, S + i] = nxt
        if ids.is_cuda:
            torch.cuda.synchronize(ids.device)
        t2 = time.perf_counter()
        self.stats = {"prefill_s": t1 - t0, "decode_s": t2 - t1,
                      "prefill_tokens_per_s": B * S / max(t1 - t0, 1e-9),
                      "decode_tokens_per_s": B * max(0, max_new_tokens - 1) / max(t2 - t1, 1e-9)}
        return out
