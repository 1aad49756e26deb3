"""The transformer plugin on CPU: reference unit assertions (plugins/model-transformer/src/lib.rs
tests), agreement with the native CPU oracle, checkpoint round trips in all three formats, and
generation with the paged KV cache against full recomputation."""
import io
import os

import numpy as np
import pytest
import torch

from coeus_b200.checkpoint.formats import load_gguf, load_safetensors
from coeus_b200.core.model import BasicGenerationConfig
from coeus_b200.foundation.error import ConfigError, ProcessingError
from coeus_b200.foundation.types import Version
from coeus_b200.models.config import DecoderConfig, Transformer250MConfig
from coeus_b200.models.decoder import DecoderLM
from coeus_b200.ops import elementwise as E
from coeus_b200.ops import norm as N
from coeus_b200.plugins.builtin import TransformerModel, TransformerModelPlugin
from coeus_b200.utils import native

SMALL = Transformer250MConfig(hidden_dim=64, num_layers=2, num_heads=2, intermediate_dim=128,
                              vocab_size=301, max_seq_len=32)


@pytest.fixture(scope="module")
def model():
    return TransformerModelPlugin().create_builder(device="cpu").build(SMALL)


def _oracle(model, ids, ref_compat=False, all_positions=False):
    c = model.decoder_config()
    flat = model._reference_flat().numpy()
    return native.module().oracle_forward(flat, c.hidden_dim, c.num_layers, c.num_heads,
                                          c.intermediate_dim, c.vocab_size, c.max_seq_len,
                                          c.norm_eps, c.use_bias, np.array(ids, dtype=np.int64),
                                          ref_compat, all_positions)


def test_plugin_identity():
    p = TransformerModelPlugin()
    assert p.id() == "transformer_model" and p.version() == Version(0, 1, 0)
    for f in ("model_building", "transformer", "250M_params"):
        assert p.capabilities().has_feature(f)


def test_forward_matches_oracle(model):
    logits = np.array(model.forward([1, 2, 3]))
    assert logits.shape == (301,)
    assert np.abs(logits - _oracle(model, [1, 2, 3])).max() < 1e-5
    # at S = 1 the reference's whole-buffer layer norm equals the per-token one
    assert np.abs(np.array(model.forward([7])) - _oracle(model, [7], ref_compat=True)).max() < 1e-5
    full = model.forward_batch([[1, 2, 3, 4]])[0].float().numpy()
    assert np.abs(full - _oracle(model, [1, 2, 3, 4], all_positions=True).reshape(4, 301)).max() < 1e-5


def test_input_validation(model):
    with pytest.raises(ProcessingError) as e:
        model.forward([1, 301])
    assert "Token ID 301 out of range [0, 300]" in str(e.value)
    with pytest.raises(ProcessingError) as e:
        model.forward(list(range(33)))
    assert "Sequence length 33 out of range [1, 32]" in str(e.value)
    with pytest.raises(ProcessingError):
        model.forward([])
    with pytest.raises(ConfigError):
        TransformerModelPlugin().create_builder(device="cpu").build(
            Transformer250MConfig(hidden_dim=65, num_heads=2))


def test_parameter_counts(model):
    assert model.num_parameters() == SMALL.buffer_parameters()
    c = Transformer250MConfig()
    assert 160_000_000 < c.buffer_parameters() < 170_000_000


def test_sin_init_matches_oracle(model):
    flat = model._reference_flat().numpy()
    want = native.module().oracle_sin_init(flat.size, 64)
    assert np.abs(flat - want).max() < 1e-6
    big = torch.empty(64)
    E.sin_init_(big, 768, index_offset=40_000_000)
    idx = (np.arange(64) + 40_000_000).astype(np.float32)   # `i as f32` loses precision here
    ref = np.clip(np.sin(idx * np.float32(0.1234567)) * np.float32(np.sqrt(2 / 768)), -0.1, 0.1)
    assert np.abs(big.numpy() - ref).max() < 1e-6


def test_math_unit_values():
    x = torch.arange(1, 9, dtype=torch.float32)[None]
    y, _, _ = N.norm_fwd(x, torch.ones(8), torch.zeros(8), 1e-5)
    assert abs(float(y.mean())) < 1e-5 and abs(float(y.var(unbiased=False)) - 1) < 1e-3
    g = E.gelu_fwd(torch.tensor([0.0, 1.0, -1.0]))
    assert g[0] == 0 and g[1] > 0.8 and g[2] < -0.1
    s = E.softmax_rows(torch.tensor([[1.0, 2.0, 3.0]]))[0]
    assert abs(float(s.sum()) - 1) < 1e-6 and s[0] < s[1] < s[2]
    pe = E.sinusoid_table(4, 8, "cpu")
    assert not torch.equal(pe[0], pe[1]) and pe[0, 0] == 0 and pe[0, 1] == 1


def test_rustllm_roundtrip_is_byte_exact(model, tmp_path):
    b = io.BytesIO()
    model.write_to(b)
    data = b.getvalue()
    assert data[:8] == b"RUSTLLM\x00" and len(data) > 136 + 4 * model.num_parameters()
    m2 = TransformerModel.read_from(io.BytesIO(data), device="cpu")
    assert m2.forward([1, 2, 3]) == model.forward([1, 2, 3])
    b2 = io.BytesIO()
    m2.write_to(b2)
    assert b2.getvalue() == data
    p = tmp_path / "m.rustllm"
    model.save(str(p))
    assert p.read_bytes() == data
    # flip one parameter byte: the checksum must catch it
    bad = bytearray(data)
    bad[136 + 40] ^= 0x01
    with pytest.raises(ProcessingError) as e:
        TransformerModel.read_from(io.BytesIO(bytes(bad)), device="cpu")
    assert "Checksum mismatch" in str(e.value)


@pytest.mark.parametrize("fmt", ["safetensors", "gguf"])
def test_named_tensor_formats(model, tmp_path, fmt):
    p = str(tmp_path / f"m.{fmt}")
    model.save(p)
    tensors, meta = (load_safetensors if fmt == "safetensors" else load_gguf)(p)
    assert meta["hidden_dim"] == "64" and meta["intermediate_dim"] == "128"
    assert tuple(tensors["token_embed"].shape) == (301, 64)
    assert tuple(tensors["layers.0.attn.q_weights"].shape) == (64, 64)
    assert tuple(tensors["layers.1.ff.up_weights"].shape) == (64, 128)
    assert tuple(tensors["output_proj"].shape) == (64, 301)
    m2 = TransformerModel.load(p, device="cpu")
    assert np.abs(np.array(m2.forward([5, 6])) - np.array(model.forward([5, 6]))).max() < 1e-6
    if fmt == "safetensors":
        from safetensors.numpy import load_file   # independent reader of the same file
        other = load_file(p)
        assert np.array_equal(other["final_ln_scale"], tensors["final_ln_scale"].numpy())
    else:
        import gguf
        r = gguf.GGUFReader(p)
        names = {t.name for t in r.tensors}
        assert "token_embed" in names and "layers.0.ff.down_weights" in names


def test_generate_with_kv_cache_equals_recomputation(model):
    out = model.generate([1, 2, 3], BasicGenerationConfig(max_length=9, temperature=0.0))
    seq = [1, 2, 3]
    for _ in range(6):
        seq.append(int(np.argmax(model.forward(seq))))
    assert out == seq
    sampled = model.generate([1, 2, 3], BasicGenerationConfig(max_length=8, temperature=0.8,
                                                              top_k=20, top_p=0.9), seed=1)
    assert len(sampled) == 8 and sampled[:3] == [1, 2, 3]


def test_llama_style_config_on_cpu():
    cfg = DecoderConfig(hidden_dim=64, num_layers=2, num_heads=2, intermediate_dim=96,
                        vocab_size=128, max_seq_len=32, use_bias=False, activation="swiglu",
                        norm="rmsnorm", pos="rope")
    m = TransformerModelPlugin().create_builder(device="cpu", init="normal").build(cfg)
    out = m.generate([3, 4, 5], BasicGenerationConfig(max_length=8, temperature=0.0))
    seq = [3, 4, 5]
    for _ in range(5):
        seq.append(int(np.argmax(m.forward(seq))))
    assert out == seq


def test_gradient_accumulation_and_schedule():
    """Two micro-batches with grad_accum=2 equal one step on their union; the schedule drives the
    optimizer's learning rate."""
    import torch
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.optim.lr import WarmupCosine
    from coeus_b200.train.trainer import TrainConfig, Trainer
    cfg = DecoderConfig(hidden_dim=32, num_layers=2, num_heads=2, intermediate_dim=64,
                        vocab_size=64, max_seq_len=16)
    torch.manual_seed(0)
    ids = torch.randint(0, 64, (4, 16))
    tgt = torch.randint(0, 64, (4, 16))
    a = Trainer(DecoderLM(cfg, "cpu", seed=1, dtype=torch.float32),
                TrainConfig(learning_rate=1e-2, eps=1.0, weight_decay=0.0))
    a.train_step(ids, tgt)
    b = Trainer(DecoderLM(cfg, "cpu", seed=1, dtype=torch.float32),
                TrainConfig(learning_rate=1e-2, eps=1.0, weight_decay=0.0, grad_accum=2))
    b.train_step(ids[:2], tgt[:2])
    assert b.step_index == 0 and torch.equal(b.model.p32, DecoderLM(cfg, "cpu", seed=1, dtype=torch.float32).p32)
    b.train_step(ids[2:], tgt[2:])
    assert b.step_index == 1
    assert (a.model.p32 - b.model.p32).abs().max() < 1e-6
    sched = WarmupCosine(peak=1e-2, warmup=2, total=10, floor=1e-3)
    assert sched.at(0) == 5e-3 and sched.at(1) == 1e-2 and abs(sched.at(10) - 1e-3) < 1e-12
    assert sched.at(5) < sched.at(3) < sched.at(2)
    c = Trainer(DecoderLM(cfg, "cpu", seed=1, dtype=torch.float32), TrainConfig(), schedule=sched)
    c.train_step(ids, tgt)
    assert c.opt.learning_rate() == 5e-3
    c.train_step(ids, tgt)
    assert c.opt.learning_rate() == 1e-2


@pytest.mark.parametrize("kind", ["gpt", "llama", "moe"])
def test_activation_recompute_gives_the_same_gradients(kind):
    import torch
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.models.decoder import DecoderLM
    kw = dict(hidden_dim=32, num_layers=3, num_heads=2, intermediate_dim=64, vocab_size=64,
              max_seq_len=16)
    if kind != "gpt":
        kw.update(use_bias=False, activation="swiglu", norm="rmsnorm", pos="rope")
    if kind == "moe":
        kw.update(num_experts=4, top_k=2, capacity_factor=2.0)
    cfg = DecoderConfig(**kw)
    torch.manual_seed(0)
    ids = torch.randint(0, 64, (2, 16))
    tgt = torch.randint(0, 64, (2, 16))
    grads = []
    for rc in (False, True):
        m = DecoderLM(cfg, "cpu", seed=3, dtype=torch.float32, recompute=rc)
        m.zero_grad()
        loss = m.forward_loss(ids, tgt)
        if rc:
            assert all(set(m._saved[l]) == {"x"} for l in m.layer_ids)
        m.backward()
        grads.append((float(loss), m.g32.clone()))
    assert grads[0][0] == grads[1][0]
    assert torch.equal(grads[0][1], grads[1][1])


def test_counter_based_normal_init():
    import numpy as np
    import torch
    from coeus_b200.ops import elementwise as E
    full = E.normal_init_(torch.empty(40_001), seed=1234, std=0.02)
    assert abs(float(full.mean())) < 5e-4 and abs(float(full.std()) - 0.02) < 5e-4
    # kurtosis of a normal distribution, and no repeated values
    z = (full / 0.02).double()
    assert abs(float((z ** 4).mean()) - 3.0) < 0.15
    assert np.unique(full.numpy()).size > 39_900
    # any slice draws what the whole tensor has there
    for off, n in ((0, 7), (5, 1), (6, 1031), (4096, 4)):
        part = E.normal_init_(torch.empty(n), seed=1234, std=0.02, index_offset=off)
        assert torch.equal(part, full[off:off + n])
    assert not torch.equal(E.normal_init_(torch.empty(64), seed=1235), full[:64])
    # known-answer test of the generator: Philox4x32-10, counter 0, key 0 (Random123 vectors)
    w = E._philox4x32(np.zeros(1, np.uint64), np.zeros(1, np.uint64), 0)
    assert [int(x[0]) for x in w] == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]


def test_philox_model_init_is_shard_invariant():
    import torch
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.models.decoder import DecoderLM
    cfg = DecoderConfig(hidden_dim=32, num_layers=4, num_heads=2, intermediate_dim=64,
                        vocab_size=64, max_seq_len=16)
    whole = DecoderLM(cfg, "cpu", init="philox", seed=2, dtype=torch.float32)
    stage = DecoderLM(cfg, "cpu", init="philox", seed=2, dtype=torch.float32, layers=(2, 4),
                      embed=False)
    for name, t in stage.named_parameters():
        assert torch.equal(t, whole.master[name]), name
    w = whole.master["layers.0.attn.qkv_weights"]
    assert abs(float(w.std()) - cfg.init_std) < 0.1 * cfg.init_std


def test_trainer_checkpoint_bytes_round_trip():
    import torch
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.train.trainer import TrainConfig, Trainer
    cfg = DecoderConfig(hidden_dim=32, num_layers=2, num_heads=2, intermediate_dim=64,
                        vocab_size=64, max_seq_len=16)
    torch.manual_seed(0)
    ids = torch.randint(0, 64, (2, 16))
    tgt = torch.randint(0, 64, (2, 16))
    a = Trainer(DecoderLM(cfg, "cpu", seed=1, dtype=torch.float32), TrainConfig(learning_rate=1e-2))
    a.train_step(ids, tgt)
    blob = a.checkpoint()
    b = Trainer(DecoderLM(cfg, "cpu", seed=9, dtype=torch.float32), TrainConfig(learning_rate=1e-2))
    b.restore(blob)
    assert b.step_index == 1 and torch.equal(a.model.p32, b.model.p32)
    la, lb = a.train_step(ids, tgt), b.train_step(ids, tgt)
    assert float(la) == float(lb) and torch.equal(a.model.p32, b.model.p32)
    with pytest.raises(Exception):
        b.restore(blob[:-4])


def test_trainer_evaluate_reports_loss_and_perplexity():
    import math
    import torch
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.train.trainer import TrainConfig, Trainer
    cfg = DecoderConfig(hidden_dim=32, num_layers=2, num_heads=2, intermediate_dim=64,
                        vocab_size=64, max_seq_len=16)
    torch.manual_seed(0)
    data = [(torch.randint(0, 64, (2, 16)), torch.randint(0, 64, (2, 16))) for _ in range(3)]
    tr = Trainer(DecoderLM(cfg, "cpu", seed=1, dtype=torch.float32), TrainConfig(learning_rate=1e-2))
    before = tr.model.p32.clone()
    ev = tr.evaluate(data)
    assert torch.equal(before, tr.model.p32) and ev["tokens"] == 96
    want = sum(float(tr.model.forward_loss(i, t)) for i, t in data) / 3
    assert abs(ev["loss"] - want) < 1e-5 and abs(ev["perplexity"] - math.exp(want)) < 1e-2
    # an untrained model is near the uniform distribution
    assert abs(ev["loss"] - math.log(64)) < 0.2
    for _ in range(30):
        tr.train_step(*data[0])
    assert tr.evaluate(data[:1])["loss"] < ev["loss"] - 0.5


def test_weight_only_quantisation():
    import torch
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.models.quant import QuantConfig, dequantize_matrix, quantize_matrix
    from coeus_b200.prelude import TransformerModelPlugin
    torch.manual_seed(0)
    w = torch.randn(64, 48) * 0.02
    for bits, group in ((8, 0), (4, 16), (8, 20)):
        codes, scales = quantize_matrix(w, bits, group)
        assert codes.dtype == torch.int8 and int(codes.abs().max()) <= 2 ** (bits - 1) - 1
        back = dequantize_matrix(codes, scales, group)
        # round to nearest: at most half a step per element
        g = 64 if group == 0 else group
        step = scales[torch.arange(64) // g]
        assert bool(((back - w).abs() <= 0.5 * step + 1e-9).all())
        # a matrix on the grid is a fixed point
        c2, s2 = quantize_matrix(back, bits, group)
        assert torch.allclose(dequantize_matrix(c2, s2, group), back, atol=1e-8)
    cfg = DecoderConfig(hidden_dim=32, num_layers=2, num_heads=2, intermediate_dim=64,
                        vocab_size=64, max_seq_len=16)
    model = TransformerModelPlugin().create_builder(device="cpu", init="normal").build(cfg)
    ids = [1, 5, 9, 33]
    before = torch.tensor(model.forward(ids))
    assert not model.is_quantized()
    model.quantize(QuantConfig(bits=8))
    assert model.is_quantized()
    after = torch.tensor(model.forward(ids))
    assert (before - after).abs().max() < 0.02 * before.abs().max() + 1e-3
    names = set(model.quantized_tensors)
    assert "layers.0.attn.qkv_weights" in names and "token_embed" not in names
    assert all(c.dtype == torch.int8 for c, _ in model.quantized_tensors.values())
    with pytest.raises(Exception):
        model.quantize(QuantConfig(bits=1))


def test_dropout_rates_are_validated_and_other_plans_refuse_them():
    from coeus_b200.models.config import DecoderConfig
    cfg = DecoderConfig(hidden_dim=32, num_layers=1, num_heads=2, intermediate_dim=64,
                        vocab_size=64, max_seq_len=16, dropout=0.1, attention_dropout=0.2)
    cfg.validate()
    with pytest.raises(Exception):
        DecoderConfig(hidden_dim=32, num_layers=1, num_heads=2, intermediate_dim=64,
                      vocab_size=64, max_seq_len=16, dropout=1.0).validate()
    with pytest.raises(Exception) as e:
        cfg.require_no_dropout("tensor parallelism")
    assert "Dropout" in str(e.value)


@pytest.mark.parametrize("kind", ["gpt", "llama_gqa"])
def test_dropout_trains_with_recomputed_masks_and_matches_autograd(kind):
    """Hidden and attention dropout in a training pass: the loss and every gradient equal an
    autograd pass through the fp32 restatement that applies the SAME masks (they are a function
    of the key and the element index), evaluation passes see no dropout, and a new step draws
    new masks."""
    import torch
    import torch.nn.functional as F
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.ops import elementwise as E
    kw = dict(hidden_dim=32, num_layers=2, num_heads=4, intermediate_dim=64, vocab_size=64,
              max_seq_len=16, dropout=0.25, attention_dropout=0.125)
    if kind == "llama_gqa":
        kw.update(num_kv_heads=2, use_bias=False, activation="swiglu", norm="rmsnorm", pos="rope")
    cfg = DecoderConfig(**kw)
    m = DecoderLM(cfg, "cpu", seed=3, dtype=torch.float32)
    ids = torch.randint(0, 64, (2, 9), generator=torch.Generator().manual_seed(0))
    x, y = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
    B, S, H, nh, dh = 2, 8, 32, 4, 8
    m.zero_grad()
    loss = m.forward_loss(x, y)
    call = m._drop_call
    m.backward()

    # the same model under autograd, masks from the same keys
    params = {n: t.clone().requires_grad_(True) for n, t in m.named_parameters()}
    from coeus_b200.models import torch_reference as R
    ln = cfg.norm == "layernorm"
    n1n, n2n, fn = ("ln1", "ln2", "final_ln") if ln else ("norm1", "norm2", "final_norm")

    def norm(t, prefix):
        if ln:
            return F.layer_norm(t, (H,), params[prefix + "_scale"], params[prefix + "_bias"],
                                cfg.norm_eps)
        return t * torch.rsqrt((t * t).mean(-1, keepdim=True) + cfg.norm_eps) * params[prefix + "_scale"]

    def key(l, site):
        return E.dropout_key(m.dropout_seed, 0, call, 0, l, site)

    def drop(t2d, rate, l, site):
        thr = E.dropout_threshold(rate)
        keep = E.dropout_mask(t2d.shape[0], t2d.shape[1], thr, key(l, site))
        return torch.where(keep, t2d * (256.0 / (256 - thr)), torch.zeros(()))

    h = params["token_embed"][x.reshape(-1)]
    if cfg.pos == "sinusoidal":
        h = h + R.sinusoid(S, H, "cpu").repeat(B, 1)
    Hkv = cfg.kv_dim
    for l in range(cfg.num_layers):
        p = f"layers.{l}."
        qkv = norm(h, p + n1n) @ params[p + "attn.qkv_weights"]
        if cfg.use_bias:
            qkv = qkv + params[p + "attn.qkv_bias"]
        q = qkv[:, :H].reshape(B, S, nh, dh)
        k = qkv[:, H:H + Hkv].reshape(B, S, cfg.kv_heads, dh)
        v = qkv[:, H + Hkv:].reshape(B, S, cfg.kv_heads, dh)
        if cfg.pos == "rope":
            q, k = R._rope(q, S, cfg.rope_theta), R._rope(k, S, cfg.rope_theta)
        g = nh // cfg.kv_heads
        k, v = k.repeat_interleave(g, 2), v.repeat_interleave(g, 2)
        sc = (q.transpose(1, 2) @ k.transpose(1, 2).transpose(-1, -2)) / dh ** 0.5
        sc = sc.masked_fill(~torch.ones(S, S, dtype=torch.bool).tril(), float("-inf"))
        pr = torch.softmax(sc, -1)
        pr = drop(pr.reshape(B * nh * S, S), cfg.attention_dropout, l, 2).reshape(B, nh, S, S)
        a = (pr @ v.transpose(1, 2)).transpose(1, 2).reshape(B * S, H)
        o = a @ params[p + "attn.o_weights"]
        if cfg.use_bias:
            o = o + params[p + "attn.o_bias"]
        h = h + drop(o, cfg.dropout, l, 0)
        n2 = norm(h, p + n2n)
        if cfg.activation == "swiglu":
            gu = n2 @ params[p + "ff.gate_up_weights"]
            f = (F.silu(gu[:, :64]) * gu[:, 64:]) @ params[p + "ff.down_weights"]
        else:
            u = n2 @ params[p + "ff.up_weights"] + params[p + "ff.up_bias"]
            f = R.gelu_tanh(u) @ params[p + "ff.down_weights"] + params[p + "ff.down_bias"]
        h = h + drop(f, cfg.dropout, l, 1)
    logits = norm(h, fn) @ params["output_proj"]
    want = F.cross_entropy(logits[:, :64], y.reshape(-1))
    want.backward()
    assert abs(float(loss) - float(want.detach())) < 1e-5
    for n, t in params.items():
        got = m.g[n]
        assert (got - t.grad).abs().max() <= 1e-4 * max(1.0, float(t.grad.abs().max())), n

    # dropout really acted, evaluation sees none, and the next step draws other masks
    m.train(False)
    plain = float(m.forward_loss(x, y))
    m.train(True)
    assert abs(plain - float(loss)) > 1e-4
    again = float(m.forward_loss(x, y))          # same step, next call: other masks
    assert abs(again - float(loss)) > 1e-6
    lg1 = m.forward_logits(x)
    lg2 = m.forward_logits(x)
    assert torch.equal(lg1, lg2)                 # inference entry points: never any dropout


def test_grouped_query_attention_trains_saves_and_serves():
    """GQA through the rest of the stack: finite-difference check of the narrow K/V gradients,
    SafeTensors round trip, chunked prefill and the batcher."""
    import torch
    from coeus_b200.checkpoint.formats import load_model, save_model
    from coeus_b200.infer.engine import InferenceEngine
    from coeus_b200.infer.scheduler import ContinuousBatcher
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.models.decoder import DecoderLM
    cfg = DecoderConfig(hidden_dim=32, num_layers=2, num_heads=4, num_kv_heads=2,
                        intermediate_dim=64, vocab_size=64, max_seq_len=160, use_bias=True)
    lm = DecoderLM(cfg, "cpu", seed=1, dtype=torch.float32)
    assert lm.master["layers.0.attn.qkv_weights"].shape == (32, 32 + 2 * 16)
    assert lm.master["layers.0.attn.qkv_bias"].shape == (64,)
    torch.manual_seed(0)
    ids, tgt = torch.randint(0, 64, (2, 16)), torch.randint(0, 64, (2, 16))
    lm.zero_grad()
    lm.forward_loss(ids, tgt)
    lm.backward()
    g = lm.g["layers.0.attn.qkv_weights"].clone()
    d = torch.zeros_like(g)
    d[:, 32:] = torch.randn(32, 32)               # a direction inside the K and V columns
    eps = 3e-3
    w = lm.master["layers.0.attn.qkv_weights"]
    base = w.clone()
    vals = []
    for sgn in (1, -1):
        w.copy_(base + sgn * eps * d)
        lm.sync_working_copy()
        vals.append(float(lm.forward_loss(ids, tgt)))
    w.copy_(base)
    lm.sync_working_copy()
    fd = (vals[0] - vals[1]) / (2 * eps)
    assert abs(fd - float((g * d).sum())) < 2e-3 * max(1.0, abs(fd))
    import tempfile, os
    path = os.path.join(tempfile.mkdtemp(), "gqa.safetensors")
    save_model(lm, path)
    back, _ = load_model(path, device="cpu")
    assert back.cfg.num_kv_heads == 2 and torch.equal(back.p32, lm.p32)
    with pytest.raises(Exception):
        save_model(lm, path.replace(".safetensors", ".rustllm"))
    prompt = torch.randint(0, 64, (1, 96))
    one = InferenceEngine(lm, max_batch=1).prefill(prompt, 128)
    chunked = InferenceEngine(lm, max_batch=1).prefill(prompt, 128, token_chunk=32)
    assert (one - chunked).abs().max() < 1e-4
    alone = InferenceEngine(lm, max_batch=1).generate(prompt[:, :70], 4)[0, 70:].tolist()
    cb = ContinuousBatcher(InferenceEngine(lm, max_batch=2), max_seqs=2, max_len=160,
                           prefix_cache=True)
    rid = cb.submit(prompt[0, :70].tolist(), 4)
    a = cb.run()[rid]
    rid = cb.submit(prompt[0, :70].tolist(), 4)              # second time through cached pages
    b = cb.run()[rid]
    assert a == alone and b == alone and cb.prefix.hits == 1


@pytest.mark.parametrize("tie", [False, True])
def test_lm_head_in_vocabulary_slices_matches_the_whole_head(tie):
    """The LM head and loss computed in slices of the vocabulary (the logits never held at once)
    give the loss and the gradients of the whole-head path."""
    cfg = DecoderConfig(vocab_size=1000, hidden_dim=64, num_layers=2, num_heads=4,
                        intermediate_dim=128, max_seq_len=32, tie_embeddings=tie)
    torch.manual_seed(0)
    ids = torch.randint(0, 1000, (2, 17))
    tg = ids[:, 1:].clone()
    tg[0, 3] = -100
    out = []
    for chunks in (1, 3):
        m = DecoderLM(cfg, device="cpu", seed=1, dtype=torch.float32, lm_head_chunks=chunks)
        m.zero_grad()
        loss = m.forward_loss(ids[:, :-1], tg)
        m.backward()
        out.append((loss.clone(), m.g32.clone()))
    assert len(m._head_chunks()) == 2
    assert torch.allclose(out[0][0], out[1][0], atol=1e-6)
    assert (out[0][1] - out[1][1]).abs().max() < 1e-6
