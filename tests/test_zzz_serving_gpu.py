"""Continuous batching on the GPU: requests of different lengths sharing decode steps get the
tokens they get when run alone (greedy)."""
import pytest
import torch

from coeus_b200.infer.engine import InferenceEngine
from coeus_b200.infer.scheduler import ContinuousBatcher
from coeus_b200.models.config import DecoderConfig
from coeus_b200.models.decoder import DecoderLM
from coeus_b200.ops import _lib

pytestmark = pytest.mark.gpu


def test_continuous_batching_matches_single_requests():
    cfg = DecoderConfig(hidden_dim=256, num_layers=2, num_heads=2, intermediate_dim=512,
                        vocab_size=1000, max_seq_len=512, use_bias=False, activation="swiglu",
                        norm="rmsnorm", pos="rope")
    m = DecoderLM(cfg, device="cuda", training=False, seed=11)
    torch.manual_seed(5)
    prompts = [torch.randint(0, 1000, (n,)).tolist() for n in (7, 130, 33, 64, 200)]
    budgets = [6, 4, 9, 3, 5]
    # one context split in both engines, so that a row is computed by the same arithmetic alone
    # and in a batch
    cb = ContinuousBatcher(InferenceEngine(m, max_batch=3, decode_splits=1), max_seqs=3,
                           max_len=256)
    ids = [cb.submit(p, k) for p, k in zip(prompts, budgets)]
    out = cb.run()
    torch.cuda.synchronize()
    _lib.check_status(torch.device("cuda", 0))
    assert cb.engine.cache.pages_in_use() == 0
    agree = total = 0
    for rid, p, k in zip(ids, prompts, budgets):
        eng = InferenceEngine(m, max_batch=1, use_graph=False, decode_splits=1)
        alone = eng.generate(torch.tensor(p, device="cuda")[None], k)[0, len(p):].tolist()
        assert len(out[rid]) == k
        # bf16 near-ties may flip an arg-max; the first token of every request must agree and
        # nearly all later ones
        assert out[rid][0] == alone[0]
        agree += sum(a == b for a, b in zip(out[rid], alone))
        total += k
    assert agree >= total - 3


def test_prefix_cache_warm_equals_cold():
    """The same prompt twice through the prefix-caching batcher: the second run adopts the first
    run's pages (same bf16 keys and values the first run attended to) and must produce the same
    tokens."""
    cfg = DecoderConfig(hidden_dim=256, num_layers=2, num_heads=2, intermediate_dim=512,
                        vocab_size=1000, max_seq_len=512, use_bias=False, activation="swiglu",
                        norm="rmsnorm", pos="rope")
    m = DecoderLM(cfg, device="cuda", training=False, seed=12)
    torch.manual_seed(8)
    prompt = torch.randint(0, 1000, (200,)).tolist()
    cb = ContinuousBatcher(InferenceEngine(m, max_batch=2, decode_splits=1), max_seqs=2,
                           max_len=256, prefix_cache=True)
    rid = cb.submit(prompt, 6)
    cold = cb.run()[rid]
    rid = cb.submit(prompt, 6)
    warm = cb.run()[rid]
    torch.cuda.synchronize()
    _lib.check_status(torch.device("cuda", 0))
    assert cb.prefix.hits == 1 and warm == cold
