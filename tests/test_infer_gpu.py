"""Decode-time kernels (paged KV write, decode attention, arg-max) against their PyTorch
restatements, and the generation engine against full recomputation on the GPU."""
import pytest
import torch

from coeus_b200.infer.engine import InferenceEngine
from coeus_b200.models.config import DecoderConfig
from coeus_b200.models.decoder import DecoderLM
from coeus_b200.ops import _lib
from coeus_b200.ops import decode as D

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("dh,nq,nh", [(64, 4, 4), (128, 2, 2), (64, 8, 2), (128, 4, 1)])
@pytest.mark.parametrize("splits", [1, 4])
def test_paged_decode_attention(dh, nq, nh, splits):
    """``nq`` query heads over a cache of ``nh`` key/value heads (grouped-query when fewer)."""
    torch.manual_seed(0)
    B, n_pages, max_pages = 3, 40, 8
    kc = torch.zeros(n_pages, D.PAGE, nh, dh, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    perm = torch.randperm(n_pages, device=DEV)[: B * max_pages].int().view(B, max_pages)
    lens = [1, 200, 333]
    for b, n in enumerate(lens):
        k = torch.randn(n, nh * dh, device=DEV).bfloat16()
        v = torch.randn(n, nh * dh, device=DEV).bfloat16()
        pos0 = torch.zeros(B, dtype=torch.int32, device=DEV)
        D.kv_write(k, v, kc, vc, perm[b:b + 1].contiguous(), pos0[:1], n, nh, dh)
    ctx = torch.tensor(lens, dtype=torch.int32, device=DEV)
    q = torch.randn(B, nq * dh, device=DEV).bfloat16()
    out = D.decode_attention(q, kc, vc, perm.contiguous(), ctx, nq, dh, splits=splits, nkv=nh)
    ref = D.decode_attention(q.cpu(), kc.cpu(), vc.cpu(), perm.cpu(), ctx.cpu(), nq, dh, nkv=nh)
    torch.cuda.synchronize()
    assert _lib.status_buffer(torch.device("cuda", 0)).tolist()[0] == 0
    assert (out.float().cpu() - ref.float()).abs().max() < 0.03


def test_argmax_rows():
    x = torch.randn(7, 50257, device=DEV).bfloat16()
    assert torch.equal(D.argmax_rows(x).cpu(), x.float().argmax(-1).cpu())


@pytest.mark.parametrize("kind", ["gpt", "llama", "gqa"])
def test_engine_matches_full_forward(kind):
    torch.manual_seed(0)
    if kind == "gpt":
        cfg = DecoderConfig(hidden_dim=256, num_layers=2, num_heads=4, intermediate_dim=512,
                            vocab_size=1000, max_seq_len=512)
    elif kind == "gqa":     # four query heads over one key/value head: the cache holds one head
        cfg = DecoderConfig(hidden_dim=256, num_layers=2, num_heads=4, num_kv_heads=1,
                            intermediate_dim=512, vocab_size=1000, max_seq_len=512,
                            use_bias=False, activation="swiglu", norm="rmsnorm", pos="rope")
    else:
        cfg = DecoderConfig(hidden_dim=256, num_layers=2, num_heads=2, intermediate_dim=512,
                            vocab_size=1000, max_seq_len=512, use_bias=False, activation="swiglu",
                            norm="rmsnorm", pos="rope")
    m = DecoderLM(cfg, device=DEV, training=False)
    eng = InferenceEngine(m)
    ids = torch.randint(0, cfg.vocab_size, (3, 150), device=DEV)
    logits = eng.prefill(ids, 160)[:, :cfg.vocab_size]
    ref = m.forward_logits(ids, last_only=True)
    assert (logits.float() - ref.float()).abs().max() < 0.05
    seq = ids
    for _ in range(4):
        nxt = ref.float().argmax(-1)
        step = eng.decode_step(nxt)[:, :cfg.vocab_size]
        seq = torch.cat([seq, nxt[:, None]], 1)
        ref = m.forward_logits(seq, last_only=True)
        assert (step.float() - ref.float()).abs().max() < 0.08
    out = eng.generate(ids, 8)
    assert out.shape == (3, 158) and torch.equal(out[:, :150], ids)
    torch.cuda.synchronize()
    _lib.check_status(torch.device("cuda", 0))


def test_chunked_prefill_matches_one_pass():
    torch.manual_seed(0)
    cfg = DecoderConfig(hidden_dim=256, num_layers=2, num_heads=2, intermediate_dim=512,
                        vocab_size=1000, max_seq_len=512, use_bias=False, activation="swiglu",
                        norm="rmsnorm", pos="rope")
    m = DecoderLM(cfg, device=DEV, training=False)
    ids = torch.randint(0, cfg.vocab_size, (3, 384), device=DEV)
    ref_eng = InferenceEngine(m)
    ref = ref_eng.prefill(ids, 400).float()
    ref_next = ref_eng.decode_step(ref.argmax(-1)).float()
    for seq_chunk, token_chunk in ((2, None), (None, 128), (1, 192)):
        eng = InferenceEngine(m)
        got = eng.prefill(ids, 400, seq_chunk=seq_chunk, token_chunk=token_chunk).float()
        assert (got - ref).abs().max() < 0.05, (seq_chunk, token_chunk)
        nxt = eng.decode_step(ref.argmax(-1)).float()
        assert (nxt - ref_next).abs().max() < 0.08, (seq_chunk, token_chunk)
    torch.cuda.synchronize()
    _lib.check_status(torch.device("cuda", 0))
