"""A small completion server: one worker thread drives the continuous batcher, HTTP handlers
hand it requests and wait for their results.

``ServingLoop`` is usable without HTTP (``submit`` returns a ``concurrent.futures.Future``);
``create_app`` wraps it in a FastAPI application with ``POST /v1/completions``,
``GET /health`` and ``GET /metrics`` (Prometheus text).  The reference names an
``InferenceService`` with ``InferenceRequest{tokens, max_length}`` and ``HealthCheck`` /
``Metrics`` traits (src/domain/inference/mod.rs:6-32, src/core/traits.rs:197-221) and has no
server; this is the deployment surface those names imply.
"""
from __future__ import annotations

import threading
import time
from concurrent.futures import Future
from typing import Dict, List, Optional

from ..core.traits import HealthCheck, Metrics
from ..foundation.error import ProcessingError
from ..infer.engine import InferenceEngine
from ..infer.scheduler import ContinuousBatcher

try:        # the request schema lives at module level so that FastAPI can resolve its annotation
    from pydantic import BaseModel, Field

    class CompletionRequest(BaseModel):
        prompt: Optional[str] = None
        prompt_ids: Optional[List[int]] = None
        max_tokens: int = Field(16, ge=1)
        temperature: float = 0.0
        top_k: Optional[int] = None
        top_p: Optional[float] = None
        eos_id: Optional[int] = None
        min_p: Optional[float] = None
        repetition_penalty: float = 1.0
        stop_ids: Optional[List[int]] = None
        stream: bool = False
except ImportError:      # ServingLoop works without the HTTP stack
    CompletionRequest = None


class ServingLoop(Metrics, HealthCheck):
    """Owns the batcher; all model work happens on its thread.  Implements the reference's
    ``Metrics`` and ``HealthCheck`` traits (src/core/traits.rs:197-221)."""

    def __init__(self, model, max_seqs: int = 16, max_len: Optional[int] = None,
                 token_chunk: Optional[int] = None, idle_sleep_s: float = 0.002,
                 prefix_cache: bool = False, engine=None, group=None) -> None:
        """``engine``: a ready engine instead of a single-GPU one built from ``model`` (e.g. a
        :class:`coeus_b200.infer.tp_engine.TPInferenceEngine`).  ``group``: the process group of a
        tensor-parallel engine; every rank of it runs a loop, rank 0 of the group takes the
        requests and sends each iteration's submissions and cancellations to the others, so all
        ranks feed their batcher the same events in the same order and step together."""
        self.engine = engine if engine is not None else InferenceEngine(
            model, max_batch=max_seqs, use_graph=False)
        self.group = group
        self.leader = True
        if group is not None:
            import torch.distributed as dist
            self.leader = dist.get_rank(group) == 0
            self._src = dist.get_global_rank(group, 0)
        self.batcher = ContinuousBatcher(self.engine, max_seqs=max_seqs, max_len=max_len,
                                         token_chunk=token_chunk, prefix_cache=prefix_cache)
        self._lock = threading.Lock()
        self._inbox: List[tuple] = []
        self._cancel: List[Future] = []
        self._futures: Dict[int, Future] = {}
        self._t0: Dict[int, float] = {}
        self._stop = threading.Event()
        self._idle = idle_sleep_s
        self.counters = {"requests": 0, "completed": 0, "failed": 0, "generated_tokens": 0,
                         "latency_s_sum": 0.0}
        self._thread = threading.Thread(target=self._run, name="coeus-serving", daemon=True)
        self._thread.start()

    def submit(self, prompt: List[int], max_new_tokens: int, **sampling) -> Future:
        """Thread-safe; the future resolves to the list of generated token ids.  ``on_token``
        (keyword) is called on the worker thread with every token as it is produced."""
        fut: Future = Future()
        with self._lock:
            self._inbox.append((prompt, max_new_tokens, sampling, fut, time.perf_counter()))
            self.counters["requests"] += 1
        return fut

    def cancel(self, fut: Future) -> None:
        """Stop working on the request behind ``fut`` (a client that went away or timed out);
        the future is cancelled and its cache pages are freed at the next step."""
        with self._lock:
            self._cancel.append(fut)

    def healthy(self) -> bool:
        return self._thread.is_alive() and not self._stop.is_set()

    def id(self) -> str:
        return "serving-loop"

    def health(self):
        from ..utils.metrics import Health
        return Health(self.healthy(), {"active": len(self.batcher.active),
                                       "waiting": len(self.batcher.waiting),
                                       "kv_pages_in_use": self.engine.cache.pages_in_use()})

    def metrics(self):
        from ..utils.metrics import Metric
        c = self.counters
        done = max(1, c["completed"])
        return [Metric("requests", c["requests"]), Metric("completed", c["completed"]),
                Metric("failed", c["failed"]), Metric("generated_tokens", c["generated_tokens"]),
                Metric("mean_latency_s", c["latency_s_sum"] / done, "s"),
                Metric("decode_steps", self.batcher.stats["steps"])]

    def reset_metrics(self) -> None:
        for k in self.counters:
            self.counters[k] = 0.0 if k == "latency_s_sum" else 0

    def close(self) -> None:
        """Leader: ends the loop on every rank (the stop travels with the next exchange)."""
        self._stop.set()
        self._thread.join(timeout=30)

    def join(self, timeout: Optional[float] = None) -> None:
        """Block until the loop ends (what the follower ranks of a tensor-parallel group do)."""
        self._thread.join(timeout)

    def _exchange(self, events: list) -> list:
        """Tensor-parallel groups: the leader's events of this iteration, on every rank."""
        if self.group is None:
            return events
        import torch.distributed as dist
        box = [events if self.leader else None]
        dist.broadcast_object_list(box, src=self._src, group=self.group)
        return box[0]

    def _run(self) -> None:
        device = self.engine.m.device
        if device.type == "cuda":
            import torch
            torch.cuda.set_device(device)
        pending_futs: List[tuple] = []          # leader: futures of this iteration's submits
        while True:
            events: list = []
            if self.leader:
                with self._lock:
                    inbox, self._inbox = self._inbox, []
                    cancels, self._cancel = self._cancel, []
                for fut in cancels:
                    inbox = [it for it in inbox if it[3] is not fut]
                    for rid, f in list(self._futures.items()):
                        if f is fut:
                            events.append(("cancel", rid))
                            self._futures.pop(rid)
                            self._t0.pop(rid, None)
                    if not fut.done():
                        fut.cancel()
                pending_futs = []
                for prompt, n, sampling, fut, t0 in inbox:
                    cb = sampling.pop("on_token", None)
                    events.append(("submit", list(prompt), int(n), dict(sampling)))
                    pending_futs.append((fut, t0, cb))
                if self._stop.is_set():
                    events.append(("stop",))
            events = self._exchange(events)
            stop, k = False, 0
            for ev in events:
                if ev[0] == "stop":
                    stop = True
                elif ev[0] == "cancel":
                    self.batcher.cancel(ev[1])
                else:
                    fut, t0, cb = pending_futs[k] if self.leader else (None, 0.0, None)
                    k += 1
                    try:
                        rid = self.batcher.submit(ev[1], ev[2], on_token=cb, **ev[3])
                        if self.leader:
                            self._futures[rid] = fut
                            self._t0[rid] = t0
                    except Exception as e:      # a bad request fails alone (on every rank alike)
                        if self.leader:
                            self.counters["failed"] += 1
                            fut.set_exception(e)
            if stop:
                self._stop.set()
                return
            if not self.batcher.pending():
                time.sleep(self._idle)
                continue
            try:
                done = self.batcher.step()
            except Exception as e:              # a model failure fails everything in flight
                for rid, fut in self._futures.items():
                    fut.set_exception(e)
                self.counters["failed"] += len(self._futures)
                self._futures.clear()
                self._stop.set()
                return
            if not self.leader:
                continue
            for r in done:
                fut = self._futures.pop(r.id)
                if r.error is not None:
                    self._t0.pop(r.id, None)
                    self.counters["failed"] += 1
                    fut.set_exception(r.error)
                    continue
                self.counters["completed"] += 1
                self.counters["generated_tokens"] += len(r.output)
                self.counters["latency_s_sum"] += time.perf_counter() - self._t0.pop(r.id)
                fut.set_result(list(r.output))


def _decoder(tokenizer):
    """ids -> text with the tokenizer's most faithful decoding (the BPE tokenizer's default
    reproduces the reference's lossy per-byte decoding; serving wants the text back)."""
    fn = getattr(tokenizer, "decode_ids", None)
    if fn is None:
        return tokenizer.decode
    try:
        fn([], ref_compat=False)
        return lambda ids: fn(ids, ref_compat=False)
    except TypeError:
        return fn


def create_app(model, tokenizer=None, max_seqs: int = 16, max_len: Optional[int] = None,
               token_chunk: Optional[int] = None, request_timeout_s: float = 120.0,
               prefix_cache: bool = False, engine=None, group=None):
    """FastAPI application.  ``tokenizer`` (anything with ``encode(str) -> ids`` and
    ``decode_ids(ids) -> str`` or ``decode(ids) -> str``) enables text prompts; without it requests carry ``prompt_ids``."""
    import asyncio

    from fastapi import FastAPI, HTTPException
    from fastapi.responses import PlainTextResponse, StreamingResponse

    from contextlib import asynccontextmanager

    loop = ServingLoop(model, max_seqs=max_seqs, max_len=max_len, token_chunk=token_chunk,
                       prefix_cache=prefix_cache, engine=engine, group=group)

    @asynccontextmanager
    async def lifespan(_app):
        yield
        loop.close()

    app = FastAPI(title="coeus_b200", lifespan=lifespan)
    app.state.loop = loop

    async def _stream(ids, max_tokens, sampling):
        """Server-sent events: one ``data: {"token_id": ...}`` line per token, then
        ``data: [DONE]``.  Tokens cross from the worker thread through the event loop's queue."""
        import json as _json
        aloop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()
        fut = loop.submit(ids, max_tokens,
                          on_token=lambda t: aloop.call_soon_threadsafe(q.put_nowait, t),
                          **sampling)
        fut.add_done_callback(lambda f: aloop.call_soon_threadsafe(q.put_nowait, None))
        decode = _decoder(tokenizer) if tokenizer is not None else None
        while True:
            tok = await asyncio.wait_for(q.get(), request_timeout_s)
            if tok is None:
                break
            ev = {"token_id": tok}
            if decode is not None:
                ev["text"] = decode([tok])
            yield f"data: {_json.dumps(ev)}\n\n"
        err = fut.exception()
        if err is not None:
            yield f"data: {_json.dumps({'error': str(err)})}\n\n"
        yield "data: [DONE]\n\n"

    @app.post("/v1/completions")
    async def completions(req: CompletionRequest):
        if req.prompt_ids is not None:
            ids = list(req.prompt_ids)
        elif req.prompt is not None and tokenizer is not None:
            ids = [int(t) for t in tokenizer.encode(req.prompt)]
        else:
            raise HTTPException(422, "give prompt_ids, or prompt when the server has a tokenizer")
        V = loop.engine.cfg.vocab_size
        if not ids or any(t < 0 or t >= V for t in ids):
            raise HTTPException(422, f"token ids must lie in [0, {V}) and the prompt be non-empty")
        sampling = dict(eos_id=req.eos_id, temperature=req.temperature, top_k=req.top_k,
                        top_p=req.top_p, min_p=req.min_p,
                        repetition_penalty=req.repetition_penalty, stop_ids=req.stop_ids or ())
        if req.stream:
            return StreamingResponse(_stream(ids, req.max_tokens, sampling),
                                     media_type="text/event-stream")
        fut = loop.submit(ids, req.max_tokens, **sampling)
        try:
            out = await asyncio.wait_for(asyncio.wrap_future(fut), request_timeout_s)
        except asyncio.TimeoutError:
            loop.cancel(fut)
            raise HTTPException(504, "generation timed out")
        except ProcessingError as e:
            raise HTTPException(422, str(e))
        body = {"token_ids": out, "usage": {"prompt_tokens": len(ids),
                                            "completion_tokens": len(out)}}
        if tokenizer is not None:
            body["text"] = _decoder(tokenizer)(out)
        return body

    @app.get("/health")
    async def health():
        if not loop.healthy():
            raise HTTPException(503, "serving loop stopped")
        return {"status": "ok", "active": len(loop.batcher.active),
                "waiting": len(loop.batcher.waiting)}

    @app.get("/metrics", response_class=PlainTextResponse)
    async def metrics():
        c, b = loop.counters, loop.batcher
        lines = [f"coeus_{k} {v}" for k, v in c.items()]
        lines += [f"coeus_active_requests {len(b.active)}",
                  f"coeus_waiting_requests {len(b.waiting)}",
                  f"coeus_kv_pages_in_use {loop.engine.cache.pages_in_use()}",
                  f"coeus_decode_steps {b.stats['steps']}"]
        if b.prefix is not None:
            lines += [f"coeus_prefix_cache_lookups {b.prefix.lookups}",
                      f"coeus_prefix_cache_hits {b.prefix.hits}",
                      f"coeus_prefix_cache_pages {len(b.prefix)}"]
        return "\n".join(lines) + "\n"

    return app
