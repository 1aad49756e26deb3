"""The completion server on CPU: concurrent HTTP requests through the continuous batcher."""
import concurrent.futures as cf

import pytest
import torch

from coeus_b200.infer.engine import InferenceEngine
from coeus_b200.models.config import DecoderConfig
from coeus_b200.models.decoder import DecoderLM


class _ByteTok:
    def encode(self, s):
        return list(s.encode())

    def decode(self, ids):
        return bytes(int(i) % 256 for i in ids).decode("latin-1")


@pytest.fixture(scope="module")
def model():
    cfg = DecoderConfig(hidden_dim=32, num_layers=2, num_heads=2, intermediate_dim=64,
                        vocab_size=256, max_seq_len=96, use_bias=False, activation="swiglu",
                        norm="rmsnorm", pos="rope")
    return DecoderLM(cfg, "cpu", seed=4, dtype=torch.float32, training=False)


def test_serving_loop_futures(model):
    from coeus_b200.serve import ServingLoop
    loop = ServingLoop(model, max_seqs=2, max_len=96)
    try:
        prompts = [[1, 2, 3], [9] * 20, [7, 7], [100, 3, 5, 8]]
        futs = [loop.submit(p, 5) for p in prompts]
        outs = [f.result(timeout=120) for f in futs]
        for p, o in zip(prompts, outs):
            alone = InferenceEngine(model, max_batch=1).generate(torch.tensor(p)[None], 5)
            assert o == alone[0, len(p):].tolist()
        # a cancelled request stops and gives its slot and pages back
        slow = loop.submit([3, 4, 5], 80)
        import time
        time.sleep(0.05)
        loop.cancel(slow)
        for _ in range(200):
            if slow.cancelled():
                break
            time.sleep(0.01)
        assert slow.cancelled()
        assert loop.submit([3, 4, 5], 2).result(timeout=60) is not None
        assert loop.engine.cache.pages_in_use() == 0 and len(loop.batcher.free_slots) == 2
        bad = loop.submit([1] * 95, 10)           # too long: fails alone
        with pytest.raises(Exception):
            bad.result(timeout=60)
        assert loop.healthy() and loop.counters["completed"] == 5 and loop.counters["failed"] == 1
        assert loop.health().healthy and loop.health().details["kv_pages_in_use"] == 0
        ms = {m.name: m.value for m in loop.metrics()}
        assert ms["completed"] == 5 and ms["generated_tokens"] == 22 and ms["mean_latency_s"] > 0
    finally:
        loop.close()
    assert not loop.healthy()


def test_http_completions(model):
    from fastapi.testclient import TestClient
    from coeus_b200.serve import create_app
    app = create_app(model, tokenizer=_ByteTok(), max_seqs=3, max_len=96)
    with TestClient(app) as client:
        assert client.get("/health").json()["status"] == "ok"

        def ask(i):
            return client.post("/v1/completions", json={"prompt": "hello " * (i + 1),
                                                        "max_tokens": 3 + i}).json()
        with cf.ThreadPoolExecutor(4) as ex:
            res = list(ex.map(ask, range(5)))
        for i, r in enumerate(res):
            assert len(r["token_ids"]) == 3 + i and isinstance(r["text"], str)
            assert r["usage"]["prompt_tokens"] == 6 * (i + 1)
        ids = client.post("/v1/completions", json={"prompt_ids": [1, 2, 3], "max_tokens": 2})
        assert ids.status_code == 200 and len(ids.json()["token_ids"]) == 2
        assert client.post("/v1/completions", json={"max_tokens": 2}).status_code == 422
        assert client.post("/v1/completions",
                           json={"prompt_ids": [999], "max_tokens": 2}).status_code == 422
        assert client.post("/v1/completions",
                           json={"prompt_ids": [1] * 95, "max_tokens": 9}).status_code == 422
        # streaming: one event per token, in order, then the end marker
        plain = client.post("/v1/completions", json={"prompt_ids": [4, 5, 6], "max_tokens": 5})
        with client.stream("POST", "/v1/completions",
                           json={"prompt_ids": [4, 5, 6], "max_tokens": 5, "stream": True}) as r:
            assert r.status_code == 200
            events = [l[6:] for l in r.iter_lines() if l.startswith("data: ")]
        assert events[-1] == "[DONE]" and len(events) == 6
        import json
        assert [json.loads(e)["token_id"] for e in events[:-1]] == plain.json()["token_ids"]
        text = client.get("/metrics").text
        assert "coeus_completed 8" in text and "coeus_kv_pages_in_use 0" in text


def test_http_prefix_cache_metrics(model):
    from fastapi.testclient import TestClient
    from coeus_b200.serve import create_app
    app = create_app(model, max_seqs=2, max_len=96, prefix_cache=True)
    system = list(range(1, 66))                       # one full page + 1 token
    with TestClient(app) as client:
        a = client.post("/v1/completions", json={"prompt_ids": system + [7], "max_tokens": 2})
        b = client.post("/v1/completions", json={"prompt_ids": system + [9, 9], "max_tokens": 2})
        assert a.status_code == 200 and b.status_code == 200
        text = client.get("/metrics").text
        assert "coeus_prefix_cache_hits 1" in text and "coeus_prefix_cache_lookups 2" in text
