"""Hugging Face Llama naming: a randomly initialised ``LlamaForCausalLM`` (transformers) and the
decoder of this framework must agree on the logits once the weights have been converted, which
pins the rotary convention, the gate / up order, the norm epsilon and every transposition."""
import pytest
import torch

from coeus_b200.checkpoint.hf import config_from_hf, load_hf_llama, to_hf_llama

transformers = pytest.importorskip("transformers")


def _tiny(tie=False, kv_heads=4):
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=kv_heads,
                      max_position_embeddings=64,
                      rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=tie,
                      attention_bias=False, mlp_bias=False)
    torch.manual_seed(0)
    return cfg, LlamaForCausalLM(cfg).eval()


@pytest.mark.parametrize("tie", [False, True])
def test_logits_match_transformers_llama(tie):
    hf_cfg, hf = _tiny(tie)
    lm = load_hf_llama(hf.state_dict(), hf_cfg, device="cpu")
    assert lm.cfg.tie_embeddings == tie and lm.cfg.rope_theta == 10000.0
    ids = torch.randint(0, 128, (2, 33))
    with torch.no_grad():
        want = hf(ids).logits.reshape(-1, 128)
    got = lm.forward_logits(ids).reshape(66, -1)[:, :128]
    assert (got - want).abs().max() < 2e-4
    # and back: the exported state dict loads into transformers and gives the same logits
    state, fields = to_hf_llama(lm)
    from transformers import LlamaConfig, LlamaForCausalLM
    keep = {k: v for k, v in fields.items() if k not in ("architectures", "model_type")}
    again = LlamaForCausalLM(LlamaConfig(**keep)).eval()
    missing = again.load_state_dict(state, strict=False)
    assert not [k for k in missing.missing_keys if "rotary" not in k and k != "lm_head.weight"]
    with torch.no_grad():
        assert (again(ids).logits.reshape(-1, 128) - want).abs().max() < 2e-4


def test_unsupported_variants_are_refused():
    with pytest.raises(Exception):
        config_from_hf({"hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 8,
                        "num_key_value_heads": 3, "intermediate_size": 128, "vocab_size": 100})
    with pytest.raises(Exception):
        config_from_hf({"hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4,
                        "intermediate_size": 128, "vocab_size": 100, "mlp_bias": True})
    with pytest.raises(Exception) as e:
        config_from_hf({"hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4,
                        "intermediate_size": 128, "vocab_size": 100, "sliding_window": 32,
                        "max_position_embeddings": 128})
    assert "sliding-window" in str(e.value)


def test_directory_round_trip_and_transformers_can_read_it(tmp_path):
    from coeus_b200.checkpoint.hf import load_hf_dir, save_hf_dir
    hf_cfg, hf = _tiny()
    lm = load_hf_llama(hf.state_dict(), hf_cfg, device="cpu")
    save_hf_dir(lm, str(tmp_path / "m"))
    back = load_hf_dir(str(tmp_path / "m"), device="cpu")
    assert torch.equal(back.p32, lm.p32)
    from transformers import AutoModelForCausalLM
    again = AutoModelForCausalLM.from_pretrained(str(tmp_path / "m")).eval()
    ids = torch.randint(0, 128, (1, 20))
    with torch.no_grad():
        assert (again(ids).logits - hf(ids).logits).abs().max() < 2e-4


def test_logits_match_transformers_mixtral():
    """Mixture of experts: router softmax, top-2 renormalised weights and the fused expert
    tensors against ``MixtralForCausalLM`` (capacity large enough that nothing is dropped)."""
    from transformers import MixtralConfig, MixtralForCausalLM
    hf_cfg = MixtralConfig(vocab_size=128, hidden_size=64, intermediate_size=96,
                           num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4,
                           max_position_embeddings=64, rms_norm_eps=1e-5, rope_theta=10000.0,
                           num_local_experts=4, num_experts_per_tok=2, sliding_window=None,
                           tie_word_embeddings=False)
    torch.manual_seed(0)
    hf = MixtralForCausalLM(hf_cfg).eval()
    if "model.layers.0.mlp.experts.gate_up_proj" not in hf.state_dict():
        pytest.skip("this transformers version stores Mixtral experts under other names")
    lm = load_hf_llama(hf.state_dict(), hf_cfg, device="cpu")
    assert lm.cfg.num_experts == 4 and lm.cfg.top_k == 2
    ids = torch.randint(0, 128, (2, 24))
    with torch.no_grad():
        want = hf(ids).logits.reshape(-1, 128)
    got = lm.forward_logits(ids).reshape(48, -1)[:, :128]
    assert (got - want).abs().max() < 3e-4


def test_loss_and_gradients_match_transformers_autograd():
    """The hand-written backward pass against PyTorch autograd through an independent
    implementation of the same architecture."""
    hf_cfg, hf = _tiny()
    hf.train()
    lm = load_hf_llama(hf.state_dict(), hf_cfg, device="cpu", training=True)
    torch.manual_seed(3)
    ids = torch.randint(0, 128, (2, 25))
    out = hf(input_ids=ids, labels=ids)            # predicts token t+1 from position t
    out.loss.backward()
    lm.zero_grad()
    loss = lm.forward_loss(ids[:, :-1].contiguous(), ids[:, 1:].contiguous())
    lm.backward()
    assert abs(float(loss) - float(out.loss.detach())) < 1e-5
    sd = dict(hf.named_parameters())
    H = 64
    g_qkv = lm.g["layers.1.attn.qkv_weights"]
    for i, x in enumerate(("q", "k", "v")):
        want = sd[f"model.layers.1.self_attn.{x}_proj.weight"].grad.t()
        assert torch.allclose(g_qkv[:, i * H:(i + 1) * H], want, atol=2e-6), x
    assert torch.allclose(lm.g["layers.0.ff.down_weights"],
                          sd["model.layers.0.mlp.down_proj.weight"].grad.t(), atol=2e-6)
    gu = lm.g["layers.0.ff.gate_up_weights"]
    assert torch.allclose(gu[:, :128], sd["model.layers.0.mlp.gate_proj.weight"].grad.t(), atol=2e-6)
    assert torch.allclose(gu[:, 128:], sd["model.layers.0.mlp.up_proj.weight"].grad.t(), atol=2e-6)
    assert torch.allclose(lm.g["token_embed"][:128], sd["model.embed_tokens.weight"].grad, atol=2e-6)
    n1 = lm.layout.norm_names[0]
    assert torch.allclose(lm.g[f"layers.0.{n1}_scale"],
                          sd["model.layers.0.input_layernorm.weight"].grad, atol=2e-6)
    assert torch.allclose(lm.g["output_proj"][:, :128], sd["lm_head.weight"].grad.t(), atol=2e-6)


def test_greedy_generation_matches_transformers():
    """Paged KV cache, decode-time rotary positions and the stop rule against
    ``LlamaForCausalLM.generate``."""
    from coeus_b200.infer.engine import InferenceEngine
    hf_cfg, hf = _tiny()
    lm = load_hf_llama(hf.state_dict(), hf_cfg, device="cpu")
    torch.manual_seed(5)
    ids = torch.randint(0, 128, (2, 9))
    with torch.no_grad():
        want = hf.generate(ids, attention_mask=torch.ones_like(ids), max_new_tokens=12,
                           do_sample=False, pad_token_id=0, eos_token_id=None)
    got = InferenceEngine(lm, max_batch=2).generate(ids, 12)
    assert torch.equal(got, want)


@pytest.mark.parametrize("kv_heads", [2, 1])
def test_grouped_query_attention_matches_transformers(kv_heads):
    """Fewer key/value heads than query heads (grouped-query / multi-query): logits, loss,
    gradients of the narrow K/V projections and greedy generation against transformers."""
    from coeus_b200.infer.engine import InferenceEngine
    hf_cfg, hf = _tiny(kv_heads=kv_heads)
    hf.train()
    lm = load_hf_llama(hf.state_dict(), hf_cfg, device="cpu", training=True)
    assert lm.cfg.kv_heads == kv_heads and lm.master["layers.0.attn.qkv_weights"].shape == (
        64, 64 + 2 * 16 * kv_heads)
    torch.manual_seed(3)
    ids = torch.randint(0, 128, (2, 25))
    out = hf(input_ids=ids, labels=ids)
    out.loss.backward()
    lm.zero_grad()
    loss = lm.forward_loss(ids[:, :-1].contiguous(), ids[:, 1:].contiguous())
    lm.backward()
    assert abs(float(loss) - float(out.loss.detach())) < 1e-5
    sd = dict(hf.named_parameters())
    Hkv = 16 * kv_heads
    g = lm.g["layers.1.attn.qkv_weights"]
    for x, lo, hi in (("q", 0, 64), ("k", 64, 64 + Hkv), ("v", 64 + Hkv, 64 + 2 * Hkv)):
        want = sd[f"model.layers.1.self_attn.{x}_proj.weight"].grad.t()
        assert torch.allclose(g[:, lo:hi], want, atol=2e-6), x
    hf.eval()
    with torch.no_grad():
        want = hf.generate(ids[:, :9], attention_mask=torch.ones_like(ids[:, :9]),
                           max_new_tokens=8, do_sample=False, pad_token_id=0, eos_token_id=None)
    assert torch.equal(InferenceEngine(lm, max_batch=2).generate(ids[:, :9], 8), want)
    state, fields = to_hf_llama(lm)
    assert fields["num_key_value_heads"] == kv_heads
    assert torch.equal(state["model.layers.0.self_attn.k_proj.weight"],
                       hf.state_dict()["model.layers.0.self_attn.k_proj.weight"])


def test_logits_match_transformers_qwen2():
    """Qwen2-style: q/k/v biases, no output-projection bias, grouped-query attention."""
    from transformers import Qwen2Config, Qwen2ForCausalLM
    hf_cfg = Qwen2Config(vocab_size=128, hidden_size=64, intermediate_size=128,
                         num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                         max_position_embeddings=64, rms_norm_eps=1e-6, rope_theta=10000.0,
                         tie_word_embeddings=False, use_sliding_window=False)
    torch.manual_seed(0)
    hf = Qwen2ForCausalLM(hf_cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("_proj.bias"):
                p.normal_(0, 0.1)
    lm = load_hf_llama(hf.state_dict(), hf_cfg, device="cpu")
    assert lm.cfg.use_bias and lm.cfg.kv_heads == 2
    ids = torch.randint(0, 128, (2, 21))
    with torch.no_grad():
        want = hf(ids).logits.reshape(-1, 128)
    got = lm.forward_logits(ids).reshape(42, -1)[:, :128]
    assert (got - want).abs().max() < 3e-4


def test_reads_a_directory_written_by_transformers(tmp_path):
    """``save_pretrained`` output (the official SafeTensors writer) through the native reader."""
    from coeus_b200.checkpoint.hf import load_hf_dir
    hf_cfg, hf = _tiny(kv_heads=2)
    hf.save_pretrained(str(tmp_path / "hf"), safe_serialization=True)
    lm = load_hf_dir(str(tmp_path / "hf"), device="cpu")
    ids = torch.randint(0, 128, (1, 17))
    with torch.no_grad():
        want = hf(ids).logits.reshape(-1, 128)
    assert (lm.forward_logits(ids).reshape(17, -1)[:, :128] - want).abs().max() < 2e-4


def test_llama3_rope_scaling_matches_transformers():
    """Llama-3.1 style frequency scaling: logits, loss and generation past the original context
    length against transformers."""
    from transformers import LlamaConfig, LlamaForCausalLM
    from coeus_b200.infer.engine import InferenceEngine
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
               "high_freq_factor": 4.0, "original_max_position_embeddings": 16,
               "rope_theta": 10000.0}
    try:
        hf_cfg = LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=128,
                             num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                             max_position_embeddings=64, rms_norm_eps=1e-5,
                             tie_word_embeddings=False, rope_parameters=scaling)
    except TypeError:
        pytest.skip("this transformers version takes rope scaling under another name")
    torch.manual_seed(0)
    hf = LlamaForCausalLM(hf_cfg)
    lm = load_hf_llama(hf.state_dict(), hf_cfg, device="cpu", training=True)
    assert lm.cfg.rope_llama3 == (8.0, 1.0, 4.0, 16)
    ids = torch.randint(0, 128, (2, 41))
    out = hf(input_ids=ids, labels=ids)
    lm.zero_grad()
    loss = lm.forward_loss(ids[:, :-1].contiguous(), ids[:, 1:].contiguous())
    lm.backward()
    assert abs(float(loss) - float(out.loss.detach())) < 1e-5
    out.loss.backward()
    want = dict(hf.named_parameters())["model.layers.0.self_attn.q_proj.weight"].grad.t()
    assert torch.allclose(lm.g["layers.0.attn.qkv_weights"][:, :64], want, atol=2e-6)
    hf.eval()
    with torch.no_grad():
        gen = hf.generate(ids[:, :30], attention_mask=torch.ones_like(ids[:, :30]),
                          max_new_tokens=10, do_sample=False, pad_token_id=0, eos_token_id=None)
    assert torch.equal(InferenceEngine(lm, max_batch=2).generate(ids[:, :30], 10), gen)
    # the scaling survives this framework's own file format
    import os
    import tempfile
    from coeus_b200.checkpoint.formats import load_model, save_model
    path = os.path.join(tempfile.mkdtemp(), "l3.safetensors")
    save_model(lm, path)
    assert load_model(path, device="cpu")[0].cfg.rope_llama3 == (8.0, 1.0, 4.0, 16)
    assert to_hf_llama(lm)[1]["rope_scaling"]["rope_type"] == "llama3"


def _tiny_gpt2():
    cfg = transformers.GPT2Config(vocab_size=131, n_positions=48, n_embd=64, n_layer=2, n_head=4,
                                  resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    torch.manual_seed(11)
    hf = transformers.GPT2LMHeadModel(cfg).eval()
    with torch.no_grad():                     # the default init leaves biases and norms trivial
        for n, p in hf.named_parameters():
            if n.endswith(".bias") or "ln_" in n:
                p.add_(0.1 * torch.randn_like(p))
    return cfg, hf


def test_gpt2_logits_loss_and_gradients_match_transformers(tmp_path):
    """The reference architecture (LayerNorm, tanh-GELU, biases, absolute positions) with a
    trained position table and tied output projection, against ``GPT2LMHeadModel``."""
    from coeus_b200.checkpoint.hf import load_hf_dir, load_hf_gpt2
    hf_cfg, hf = _tiny_gpt2()
    lm = load_hf_gpt2(hf.state_dict(), hf_cfg, device="cpu", training=True)
    assert lm.cfg.pos == "learned" and lm.cfg.tie_embeddings
    torch.manual_seed(2)
    ids = torch.randint(0, 131, (2, 21))
    with torch.no_grad():
        want = hf(ids).logits.reshape(-1, 131)
    assert (lm.forward_logits(ids).reshape(42, -1)[:, :131] - want).abs().max() < 2e-4
    out = hf(input_ids=ids, labels=ids)
    out.loss.backward()
    lm.zero_grad()
    loss = lm.forward_loss(ids[:, :-1].contiguous(), ids[:, 1:].contiguous())
    lm.backward()
    assert abs(float(loss) - float(out.loss.detach())) < 1e-5
    sd = dict(hf.named_parameters())
    # position rows beyond the sequence get no gradient; the tied table gets both contributions
    assert torch.allclose(lm.g["pos_embed"], sd["transformer.wpe.weight"].grad, atol=2e-6)
    assert torch.allclose(lm.g["token_embed"][:131], sd["transformer.wte.weight"].grad, atol=2e-6)
    assert torch.allclose(lm.g["layers.1.attn.qkv_weights"],
                          sd["transformer.h.1.attn.c_attn.weight"].grad, atol=2e-6)
    assert torch.allclose(lm.g["layers.0.ff.up_bias"],
                          sd["transformer.h.0.mlp.c_fc.bias"].grad, atol=2e-6)
    assert torch.allclose(lm.g["final_ln_bias"], sd["transformer.ln_f.bias"].grad, atol=2e-6)
    with pytest.raises(Exception, match="[Ss]equence length"):       # 48 trained positions
        lm.forward_logits(torch.zeros(1, 49, dtype=torch.long))
    # and through the directory reader (the writer de-duplicates the tied head)
    hf.save_pretrained(str(tmp_path / "g"), safe_serialization=True)
    lm2 = load_hf_dir(str(tmp_path / "g"), device="cpu")
    assert (lm2.forward_logits(ids).reshape(42, -1)[:, :131] - want).abs().max() < 2e-4


def test_gpt2_export_is_read_by_transformers(tmp_path):
    from coeus_b200.checkpoint.hf import load_hf_dir, load_hf_gpt2, save_hf_dir
    hf_cfg, hf = _tiny_gpt2()
    lm = load_hf_gpt2(hf.state_dict(), hf_cfg, device="cpu")
    save_hf_dir(lm, str(tmp_path / "m"))
    assert torch.equal(load_hf_dir(str(tmp_path / "m"), device="cpu").p32, lm.p32)
    again = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path / "m")).eval()
    ids = torch.randint(0, 131, (1, 20))
    with torch.no_grad():
        assert (again(ids).logits - hf(ids).logits).abs().max() < 2e-4


def test_gpt2_greedy_generation_matches_transformers():
    from coeus_b200.infer.engine import InferenceEngine
    from coeus_b200.infer.scheduler import ContinuousBatcher
    from coeus_b200.checkpoint.hf import load_hf_gpt2
    hf_cfg, hf = _tiny_gpt2()
    lm = load_hf_gpt2(hf.state_dict(), hf_cfg, device="cpu")
    torch.manual_seed(5)
    ids = torch.randint(0, 131, (2, 9))
    with torch.no_grad():
        want = hf.generate(ids, attention_mask=torch.ones_like(ids), max_new_tokens=12,
                           do_sample=False, pad_token_id=0, eos_token_id=None)
    eng = InferenceEngine(lm, max_batch=2)
    assert torch.equal(eng.generate(ids, 12), want)
    # rows at different positions in one decode batch (per-row position lookups)
    cb = ContinuousBatcher(InferenceEngine(lm, max_batch=2), max_seqs=2, max_len=40)
    a = cb.submit(ids[0].tolist(), 12)
    b = cb.submit(ids[1, :5].tolist(), 6)
    out = cb.run()
    assert out[a] == want[0, 9:].tolist()
    with torch.no_grad():
        w2 = hf.generate(ids[1:2, :5], attention_mask=torch.ones(1, 5, dtype=torch.long),
                         max_new_tokens=6, do_sample=False, pad_token_id=0, eos_token_id=None)
    assert out[b] == w2[0, 5:].tolist()
