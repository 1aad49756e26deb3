"""Continuous batching: requests of different prompt lengths join and leave a running decode batch.

Every request owns one row ("slot") of the paged KV cache.  A step admits waiting requests into
free slots (their prompts are prefilled one by one, optionally in chunks), then feeds one token
per active slot through the model in a single decode batch whose rows sit at different positions
(per-row positions for RoPE, per-row context lengths for the paged attention kernel), samples,
and retires the rows that are done, returning their pages to the free list.  The reference's
``InferenceRequest{tokens, max_length}`` / ``InferenceResult{predictions}``
(src/domain/inference/mod.rs:6-32) name a request and a result; it has no batching or cache.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional

import torch

from ..foundation.error import Error, ProcessingError
from .engine import InferenceEngine
from .sampler import select


@dataclass
class Request:
    id: int
    prompt: List[int]
    max_new_tokens: int
    eos_id: Optional[int] = None
    temperature: float = 0.0
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    min_p: Optional[float] = None
    repetition_penalty: float = 1.0
    stop_ids: tuple = ()                 # further token ids that end the request like eos_id
    output: List[int] = field(default_factory=list)
    slot: int = -1
    on_token: Optional[Callable[[int], None]] = None      # called with every new token
    error: Optional[BaseException] = None                  # set when the request failed alone

    def push(self, tok: int) -> None:
        self.output.append(tok)
        if self.on_token is not None:
            self.on_token(tok)

    @property
    def done(self) -> bool:
        if len(self.output) >= self.max_new_tokens:
            return True
        if not self.output:
            return False
        last = self.output[-1]
        return (self.eos_id is not None and last == self.eos_id) or last in self.stop_ids


class PrefixCache:
    """Prompt prefixes whose keys and values are already in cache pages, by page: entry ``j`` of a
    prompt is keyed by all of its first ``64 * (j + 1)`` tokens, so two prompts share exactly the
    pages of their common page-aligned prefix.  The cache holds one reference on every page it
    knows; pages nobody else uses are given back, least recently used first, when the pool runs
    dry."""

    def __init__(self, kv) -> None:
        self.kv = kv
        # (parent entry id, the page's 64 tokens) -> [entry id, page]; the chain through the
        # parents spells the whole prefix, so a key is exact without storing the prefix again.
        # Dict order = recency (entries are re-inserted when touched).
        self.entries: "Dict[tuple, list]" = {}
        self._next = 1
        self.hits = self.lookups = 0

    def _walk(self, prompt: List[int], page: int):
        parent = 0
        for j in range(len(prompt) // page):
            yield j, (parent, tuple(prompt[page * j:page * (j + 1)]))
            e = self.entries.get((parent, tuple(prompt[page * j:page * (j + 1)])))
            if e is None:
                return
            parent = e[0]

    def match(self, prompt: List[int], page: int) -> List[int]:
        """Pages of the longest cached prefix that still leaves one prompt token to compute."""
        out = []
        for j, key in self._walk(prompt, page):
            e = self.entries.get(key)
            if e is None or page * (j + 1) >= len(prompt):
                break
            out.append(e[1])
            self.entries[key] = self.entries.pop(key)      # touch
        self.lookups += 1
        self.hits += bool(out)
        return out

    def insert(self, prompt: List[int], page: int, owned: List[int]) -> None:
        """Remember the full prompt pages of a sequence that owns ``owned`` (its pages in order)."""
        parent = 0
        for j in range(min(len(prompt) // page, len(owned))):
            key = (parent, tuple(prompt[page * j:page * (j + 1)]))
            e = self.entries.get(key)
            if e is None:
                e = [self._next, owned[j]]
                self._next += 1
                self.entries[key] = e
                self.kv.retain(owned[j])
            parent = e[0]

    def evict(self, want: int) -> int:
        """Give back up to ``want`` pages that only the cache still holds (least recently used
        first; an entry whose page goes away takes its descendants' reachability with it, they
        age out the same way); returns how many."""
        freed = 0
        for key in list(self.entries):
            if freed >= want:
                break
            pg = self.entries[key][1]
            if self.kv.refs[pg] == 1:
                del self.entries[key]
                self.kv.drop(pg)
                freed += 1
        return freed

    def __len__(self) -> int:
        return len(self.entries)


class ContinuousBatcher:
    def __init__(self, engine: InferenceEngine, max_seqs: int = 64, max_len: Optional[int] = None,
                 token_chunk: Optional[int] = None, seed: int = 0,
                 prefix_cache: bool = False) -> None:
        """``max_seqs`` rows decode together; ``max_len`` bounds prompt + generated tokens of one
        request; ``token_chunk`` prefills long prompts in pieces; ``prefix_cache`` reuses the
        cache pages of prompt prefixes that earlier requests already computed (shared system
        prompts), in units of whole pages."""
        self.engine = engine
        self.max_seqs = max_seqs
        self.max_len = max_len or engine.max_len
        self.token_chunk = token_chunk
        self.device = engine.m.device
        engine.open_slots(max_seqs, self.max_len)
        self.prefix = PrefixCache(engine.cache) if prefix_cache and hasattr(
            engine, "prefill_slot_paged") else None
        self.waiting: Deque[Request] = deque()
        self.active: Dict[int, Request] = {}          # slot -> request
        self.free_slots: List[int] = list(range(max_seqs - 1, -1, -1))
        self._next_id = 0
        self._gen = torch.Generator(device=self.device)
        self._gen.manual_seed(seed)
        self.stats = {"steps": 0, "prefills": 0, "decoded_tokens": 0, "max_active": 0}

    # ------------------------------------------------------------------ API
    def submit(self, prompt, max_new_tokens: int, eos_id: Optional[int] = None,
               temperature: float = 0.0, top_k: Optional[int] = None,
               top_p: Optional[float] = None,
               on_token: Optional[Callable[[int], None]] = None, min_p: Optional[float] = None,
               repetition_penalty: float = 1.0, stop_ids=()) -> int:
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ProcessingError.invalid_input("empty prompt")
        if len(prompt) + max_new_tokens > self.max_len:
            raise ProcessingError.limit_exceeded("sequence length", self.max_len,
                                                 len(prompt) + max_new_tokens)
        rid = self._next_id
        self._next_id += 1
        self.waiting.append(Request(rid, prompt, max_new_tokens, eos_id, temperature, top_k, top_p,
                                    min_p=min_p, repetition_penalty=repetition_penalty,
                                    stop_ids=tuple(int(t) for t in (stop_ids or ())),
                                    on_token=on_token))
        return rid

    def cancel(self, rid: int) -> bool:
        """Drop request ``rid`` wherever it is (waiting or decoding); its pages go back to the
        pool.  Returns whether it was found."""
        for r in list(self.waiting):
            if r.id == rid:
                self.waiting.remove(r)
                return True
        for r in list(self.active.values()):
            if r.id == rid:
                self.active.pop(r.slot, None)
                self.engine.cache.release(r.slot)
                self.free_slots.append(r.slot)
                return True
        return False

    def pending(self) -> int:
        return len(self.waiting) + len(self.active)

    def step(self) -> List[Request]:
        """Admit, decode one token per active request, retire; returns the requests that finished
        in this step."""
        eng, cache = self.engine, self.engine.cache
        finished: List[Request] = []
        # a request's first token comes from its prefill
        while self.waiting and self.free_slots:
            r = self.waiting.popleft()
            r.slot = self.free_slots.pop()
            ids = torch.tensor(r.prompt, dtype=torch.int64, device=self.device)
            try:
                logits = self._prefill(r, ids)
            except BaseException as e:
                # whatever the prefill raised, the slot and the pages it reserved or adopted go
                # back first; an ordinary exception (a framework error such as "no pages", a
                # kernel-library or torch error) then ends this request only, anything else
                # (KeyboardInterrupt, SystemExit) propagates
                eng.cache.release(r.slot)
                self.free_slots.append(r.slot)
                r.slot = -1
                if not isinstance(e, Exception):
                    self.waiting.appendleft(r)
                    raise
                r.error = e
                finished.append(r)
                continue
            r.push(int(self._sample(logits[None], r)[0]))
            self.stats["prefills"] += 1
            if r.done:
                self._retire(r, finished)
            else:
                self.active[r.slot] = r
        if self.active:
            order = sorted(self.active)
            reqs = [self.active[s] for s in order]
            slots = torch.tensor(order, dtype=torch.int64, device=self.device)
            tokens = torch.tensor([r.output[-1] for r in reqs], dtype=torch.int64,
                                  device=self.device)
            pos = torch.tensor([len(r.prompt) + len(r.output) - 1 for r in reqs],
                               dtype=torch.int32, device=self.device)
            logits = eng.decode_slots(slots, tokens, pos)
            greedy = all(not r.temperature and r.repetition_penalty == 1.0 for r in reqs)
            V = eng.cfg.vocab_size   # the padding columns of the vocabulary never compete
            nxt = select(logits[:, :V], 0.0, None, None, None).tolist() if greedy else None
            for i, r in enumerate(reqs):
                tok = nxt[i] if greedy else int(self._sample(logits[i:i + 1], r)[0])
                r.push(int(tok))
                cache.set_length(r.slot, len(r.prompt) + len(r.output) - 1)
                if r.done:
                    self._retire(r, finished)
            self.stats["decoded_tokens"] += len(reqs)
            self.stats["max_active"] = max(self.stats["max_active"], len(reqs))
        self.stats["steps"] += 1
        return finished

    def run(self) -> Dict[int, List[int]]:
        """Steps until nothing is pending; returns ``{request id: generated tokens}``."""
        out: Dict[int, List[int]] = {}
        while self.pending():
            for r in self.step():
                if r.error is not None:
                    raise r.error
                out[r.id] = r.output
        return out

    # ------------------------------------------------------------------ internals
    def _prefill(self, r: Request, ids: torch.Tensor) -> torch.Tensor:
        eng, total = self.engine, len(r.prompt) + r.max_new_tokens
        if self.prefix is None:
            return eng.prefill_slot(r.slot, ids, total, token_chunk=self.token_chunk)
        from ..ops.decode import PAGE
        from ..foundation.error import ResourceError
        for attempt in range(2):
            pages = self.prefix.match(r.prompt, PAGE)
            try:
                logits = eng.prefill_slot_paged(r.slot, ids, total, pages)
                break
            except ResourceError:
                # the pool is full of cached prefixes nobody uses right now: drop some, retry
                eng.cache.release(r.slot)
                if attempt or not self.prefix.evict(total // PAGE + 2):
                    raise
        self.prefix.insert(r.prompt, PAGE, eng.cache.owned[r.slot])
        return logits

    def _sample(self, logits: torch.Tensor, r: Request) -> torch.Tensor:
        V = self.engine.cfg.vocab_size
        gen = self._gen if r.temperature else None
        hist = None
        if r.repetition_penalty != 1.0:
            hist = torch.tensor([r.prompt + r.output], dtype=torch.int64, device=logits.device)
        return select(logits[:, :V], r.temperature, r.top_k, r.top_p, gen, min_p=r.min_p,
                      history=hist, repetition_penalty=r.repetition_penalty)

    def _retire(self, r: Request, finished: List[Request]) -> None:
        self.active.pop(r.slot, None)
        self.engine.cache.release(r.slot)
        self.free_slots.append(r.slot)
        finished.append(r)
