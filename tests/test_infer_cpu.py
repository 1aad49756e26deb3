"""The generation engine on CPU (the ops' oracle paths): chunked prefill against one-pass prefill,
and the paged decode against recomputing the full sequence."""
import pytest
import torch

from coeus_b200.infer.engine import InferenceEngine
from coeus_b200.models.config import DecoderConfig
from coeus_b200.models.decoder import DecoderLM


def _model(kind):
    kw = dict(hidden_dim=32, num_layers=2, num_heads=2, intermediate_dim=64, vocab_size=96,
              max_seq_len=160)
    if kind == "llama":
        kw.update(use_bias=False, activation="swiglu", norm="rmsnorm", pos="rope")
    return DecoderLM(DecoderConfig(**kw), "cpu", seed=4, dtype=torch.float32, training=False)


@pytest.mark.parametrize("kind", ["gpt", "llama"])
def test_chunked_prefill_matches_one_pass(kind):
    m = _model(kind)
    torch.manual_seed(0)
    ids = torch.randint(0, 96, (3, 96))
    ref_eng = InferenceEngine(m, max_batch=4)
    ref = ref_eng.prefill(ids, 128)
    ref_next = ref_eng.decode_step(ref.argmax(-1))
    for seq_chunk, token_chunk in ((2, None), (None, 32), (1, 40), (2, 96)):
        eng = InferenceEngine(m, max_batch=4)
        got = eng.prefill(ids, 128, seq_chunk=seq_chunk, token_chunk=token_chunk)
        assert (got - ref).abs().max() < 1e-4, (seq_chunk, token_chunk)
        # the cache the chunks wrote serves the next decode step
        nxt = eng.decode_step(ref.argmax(-1))
        assert (nxt - ref_next).abs().max() < 1e-4, (seq_chunk, token_chunk)


def test_decode_matches_full_recompute():
    m = _model("llama")
    torch.manual_seed(1)
    ids = torch.randint(0, 96, (2, 17))
    eng = InferenceEngine(m, max_batch=2)
    out = eng.generate(ids, 6)
    assert out.shape == (2, 23) and torch.equal(out[:, :17], ids)
    # an end-of-sequence token freezes its sequence; the other keeps decoding
    eos = int(out[0, 19])
    stopped = InferenceEngine(m, max_batch=2).generate(ids, 6, eos_id=eos)
    first = out[0, 17:].tolist().index(eos)
    assert stopped[0, 17:17 + first + 1].tolist() == out[0, 17:17 + first + 1].tolist()
    assert set(stopped[0, 17 + first:].tolist()) == {eos}
    if eos not in out[1, 17:].tolist():
        assert torch.equal(stopped[1], out[1])
    for i in range(6):          # greedy continuation of the full-sequence forward
        logits = m.forward_logits(out[:, :17 + i], last_only=True)[:, :96]
        assert torch.equal(logits.argmax(-1).reshape(-1), out[:, 17 + i])


@pytest.mark.parametrize("kind", ["gpt", "llama"])
def test_continuous_batching_matches_one_request_at_a_time(kind):
    """Requests with different prompt lengths and budgets share decode steps (more requests than
    slots, so rows are reused) and each gets what it would get alone."""
    from coeus_b200.infer.scheduler import ContinuousBatcher
    m = _model(kind)
    torch.manual_seed(2)
    prompts = [torch.randint(0, 96, (n,)).tolist() for n in (5, 17, 9, 30, 3, 12, 64)]
    budgets = [4, 7, 1, 5, 9, 3, 6]
    alone = []
    for p, k in zip(prompts, budgets):
        eng = InferenceEngine(m, max_batch=1)
        alone.append(eng.generate(torch.tensor(p)[None], k)[0, len(p):].tolist())
    cb = ContinuousBatcher(InferenceEngine(m, max_batch=3), max_seqs=3, max_len=128,
                           token_chunk=16)
    ids = [cb.submit(p, k) for p, k in zip(prompts, budgets)]
    out = cb.run()
    assert [out[i] for i in ids] == alone
    assert cb.stats["max_active"] == 3 and cb.stats["prefills"] == 7
    assert cb.engine.cache.pages_in_use() == 0 and len(cb.free_slots) == 3
    # an end-of-sequence token stops a request early
    first = alone[1][2]
    rid = cb.submit(prompts[1], 7, eos_id=first)
    got = cb.run()[rid]
    assert got == alone[1][:alone[1].index(first) + 1]
    rid = cb.submit(prompts[1], 7, stop_ids=[alone[1][3], alone[1][1]])
    got = cb.run()[rid]
    cut = min(alone[1].index(alone[1][3]), alone[1].index(alone[1][1]))
    assert got == alone[1][:cut + 1]
    with pytest.raises(Exception):
        cb.submit([1] * 200, 10)
    # a strong repetition penalty: no token is produced twice while unseen ones remain
    rid = cb.submit(prompts[0], 12, repetition_penalty=1e6)
    got = cb.run()[rid]
    assert len(set(got)) == len(got) and not set(got) & set(prompts[0])


def test_sampler_filters():
    from coeus_b200.infer.sampler import apply_repetition_penalty, select
    logits = torch.tensor([[4.0, 3.9, 1.0, -2.0, 0.0]])
    assert int(select(logits)) == 0
    # a penalised favourite loses to the runner-up; negative logits move further down
    hist = torch.tensor([[0, 3, -1]])
    pen = apply_repetition_penalty(logits, hist, 2.0)
    assert pen[0].tolist() == [2.0, 3.9000000953674316, 1.0, -4.0, 0.0]
    assert int(select(logits, history=hist, repetition_penalty=2.0)) == 1
    g = torch.Generator().manual_seed(0)
    draws = {int(select(logits, 1.0, min_p=0.5, generator=g)) for _ in range(200)}
    assert draws == {0, 1}                       # everything below half the top probability is cut
    draws = {int(select(logits, 1.0, top_k=3, generator=g)) for _ in range(300)}
    assert draws <= {0, 1, 2} and {0, 1} <= draws
    draws = {int(select(logits, 1.0, top_p=0.6, generator=g)) for _ in range(200)}
    assert draws == {0, 1}


@pytest.mark.parametrize("kind", ["gpt", "llama"])
def test_prefix_cache_reuses_pages_and_changes_nothing(kind):
    """Requests that share a long system prompt: with the prefix cache the shared pages are
    computed once and every request still gets exactly the tokens it gets without it."""
    from coeus_b200.infer.scheduler import ContinuousBatcher
    m = _model(kind)
    torch.manual_seed(4)
    system = torch.randint(0, 96, (130,)).tolist()           # two full pages + 2 tokens
    prompts = [system + torch.randint(0, 96, (n,)).tolist() for n in (3, 9, 1)] + \
              [system[:64] + [5, 6, 7], torch.randint(0, 96, (70,)).tolist(), system[:128]]
    budgets = [3, 2, 4, 2, 3, 2]

    def run(prefix_cache):
        cb = ContinuousBatcher(InferenceEngine(m, max_batch=2), max_seqs=2, max_len=160,
                               prefix_cache=prefix_cache)
        ids = [cb.submit(p, k) for p, k in zip(prompts, budgets)]
        out = cb.run()
        return [out[i] for i in ids], cb

    plain, _ = run(False)
    cached, cb = run(True)
    assert cached == plain
    assert cb.prefix.hits >= 4 and len(cb.prefix) >= 3
    kv = cb.engine.cache
    # nothing is active: every page in use is held by the prefix cache alone
    assert kv.pages_in_use() == len(cb.prefix) and all(kv.refs[e[1]] == 1
                                                       for e in cb.prefix.entries.values())
    assert cb.prefix.evict(100) == len(kv.refs) - len(kv.free) or kv.pages_in_use() == 0
    assert kv.pages_in_use() == 0


def test_prefix_cache_gives_pages_back_under_pressure():
    from coeus_b200.infer.scheduler import ContinuousBatcher
    m = _model("llama")
    torch.manual_seed(6)
    prompts = [torch.randint(0, 96, (140,)).tolist() for _ in range(4)]     # nothing in common
    alone = [InferenceEngine(m, max_batch=1).generate(torch.tensor(p)[None], 3)[0, 140:].tolist()
             for p in prompts]
    cb = ContinuousBatcher(InferenceEngine(m, max_batch=1), max_seqs=1, max_len=160,
                           prefix_cache=True)
    assert cb.engine.cache.num_pages == 4            # one sequence's worth of pages
    got = []
    for p in prompts:                                # each request finds the pool full of the
        rid = cb.submit(p, 3)                        # previous prompt's cached pages
        got.append(cb.run()[rid])
    assert got == alone and cb.prefix.hits == 0
    rid = cb.submit(prompts[-1] + [1, 2], 2)         # the most recent prompt is still cached
    cb.run()
    assert cb.prefix.hits == 1


def test_generation_never_picks_a_vocabulary_padding_column():
    """Vocabulary 90 is padded to 96 columns whose logits are exactly zero; with every real logit
    pushed below zero the arg-max must still be a real token."""
    from coeus_b200.infer.scheduler import ContinuousBatcher
    cfg = DecoderConfig(hidden_dim=32, num_layers=1, num_heads=2, intermediate_dim=64,
                        vocab_size=90, max_seq_len=32)
    m = DecoderLM(cfg, "cpu", seed=2, dtype=torch.float32, training=False)
    assert cfg.vocab_padded > cfg.vocab_size
    name = "token_embed" if cfg.tie_embeddings else "output_proj"
    fn = m.layout.norm_names[2]
    u = torch.linspace(0.1, 1.0, 32)
    if name == "output_proj":                              # every real column is the vector u
        m.master[name][:, :90] = u[:, None]
    else:
        m.master[name][:90] = u[None, :]
    m.master[fn + "_scale"].zero_()                        # final hidden state = the bias = -u
    m.master[fn + "_bias"].copy_(-u)                       # so every real logit is -|u|^2 < 0
    m.sync_working_copy()
    ids = torch.randint(0, 90, (2, 5))
    logits = m.forward_logits(ids, last_only=True)
    assert bool((logits[:, :90] < 0).all()) and bool((logits[:, 90:] == 0).all())
    out = InferenceEngine(m, max_batch=2).generate(ids, 3)
    assert int(out.max()) < 90
    cb = ContinuousBatcher(InferenceEngine(m, max_batch=2), max_seqs=2, max_len=32)
    rid = cb.submit(ids[0].tolist(), 3)
    assert max(cb.run()[rid]) < 90


def test_a_request_that_cannot_be_admitted_fails_alone():
    """The page pool is made too small for the second request's prompt: it fails with a resource
    error, its slot comes back, the others are served."""
    from coeus_b200.infer.scheduler import ContinuousBatcher
    m = _model("llama")
    cb = ContinuousBatcher(InferenceEngine(m, max_batch=2), max_seqs=2, max_len=160)
    kv = cb.engine.cache
    while len(kv.free) > 2:              # leave two pages in the pool
        kv.free.pop()
    ok1 = cb.submit([1, 2, 3], 2)
    big = cb.submit(list(range(1, 91)) + [5] * 60, 2)        # needs three pages
    done = {}
    errors = {}
    while cb.pending():
        for r in cb.step():
            (errors if r.error is not None else done)[r.id] = r
    assert list(done) == [ok1] and list(errors) == [big]
    assert "exhausted" in str(errors[big].error)
    assert len(cb.free_slots) == 2 and kv.pages_in_use() == kv.num_pages - 2
    ok2 = cb.submit([4, 5, 6], 2)
    assert len(cb.run()[ok2]) == 2


def test_a_prefill_that_raises_a_foreign_error_gives_its_slot_and_pages_back():
    """An exception that is not one of the framework's (a kernel-library or torch error is a
    ``RuntimeError``) ends that request only: the slot and the pages return to their pools and
    the batcher keeps serving."""
    from coeus_b200.infer.scheduler import ContinuousBatcher
    m = _model("llama")
    cb = ContinuousBatcher(InferenceEngine(m, max_batch=2), max_seqs=2, max_len=160)
    kv = cb.engine.cache
    slots0, pages0 = len(cb.free_slots), kv.pages_in_use()
    real = cb.engine.prefill_slot

    def boom(slot, ids, total, **kw):
        real(slot, ids, total, **kw)          # reserves pages and writes K/V first
        raise RuntimeError("launch failed")
    cb.engine.prefill_slot = boom
    bad = cb.submit([1, 2, 3, 4], 3)
    fin = cb.step()
    assert [r.id for r in fin] == [bad] and isinstance(fin[0].error, RuntimeError)
    assert len(cb.free_slots) == slots0 and kv.pages_in_use() == pages0
    assert cb.pending() == 0
    cb.engine.prefill_slot = real
    ok = cb.submit([4, 5, 6], 2)
    assert len(cb.run()[ok]) == 2
