"""The autograd layers on the GPU: ``nn.TransformerLM`` against the explicit decoder with the same
weights (both run the same kernels; the autograd path adds the graph and bf16 gradient tensors),
and a few steps of ``ModuleAdamW``."""
import pytest
import torch

from coeus_b200.models.config import DecoderConfig
from coeus_b200.models.decoder import DecoderLM
from coeus_b200.nn import TransformerLM
from coeus_b200.ops import _lib
from coeus_b200.optim.adamw import AdamWConfig
from coeus_b200.optim.module import ModuleAdamW

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", ["gpt", "llama"])
def test_autograd_model_matches_explicit_decoder(kind):
    kw = dict(hidden_dim=256, num_layers=2, num_heads=4, intermediate_dim=512, vocab_size=1024,
              max_seq_len=256)
    if kind == "llama":
        kw.update(use_bias=False, activation="swiglu", norm="rmsnorm", pos="rope")
    cfg = DecoderConfig(**kw)
    lm = DecoderLM(cfg, device="cuda", seed=3)
    net = TransformerLM(cfg, device="cuda")
    net.load_from(lm)
    torch.manual_seed(0)
    ids = torch.randint(0, 1024, (2, 200), device="cuda")
    tgt = torch.randint(0, 1024, (2, 200), device="cuda")
    lm.zero_grad()
    want = float(lm.forward_loss(ids, tgt))
    lm.backward()
    loss = net(ids, tgt)
    loss.backward()
    torch.cuda.synchronize()
    _lib.check_status(torch.device("cuda", 0))
    assert abs(float(loss.detach()) - want) < 0.02
    g_auto = net.blocks[1].attn.qkv.weight.grad.float()
    g_expl = lm.g["layers.1.attn.qkv_weights"]
    assert (g_auto - g_expl).abs().max() <= 0.05 * g_expl.abs().max() + 1e-4


def test_module_adamw_trains_on_gpu():
    cfg = DecoderConfig(hidden_dim=256, num_layers=2, num_heads=4, intermediate_dim=512,
                        vocab_size=1024, max_seq_len=128, use_bias=False, activation="swiglu",
                        norm="rmsnorm", pos="rope")
    net = TransformerLM(cfg, device="cuda")
    opt = ModuleAdamW(net, AdamWConfig(lr=3e-3, grad_clip=1.0))
    torch.manual_seed(1)
    ids = torch.randint(0, 1024, (4, 128), device="cuda")
    tgt = torch.roll(ids, -1, 1)
    losses = []
    for _ in range(8):
        opt.zero_grad()
        loss = net(ids, tgt)
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    torch.cuda.synchronize()
    _lib.check_status(torch.device("cuda", 0))
    assert losses[-1] < losses[0]


@pytest.mark.parametrize("kv_heads", [4, 2])
def test_gpu_decoder_matches_transformers_llama(kv_heads):
    """The bf16 kernel path against an independent fp32 implementation (transformers' Llama) of
    the same weights; with two key/value heads the grouped-query expansion is in the path."""
    transformers = pytest.importorskip("transformers")
    from coeus_b200.checkpoint.hf import load_hf_llama
    hf_cfg = transformers.LlamaConfig(
        vocab_size=1024, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
        num_attention_heads=4, num_key_value_heads=kv_heads, max_position_embeddings=256,
        rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False)
    torch.manual_seed(0)
    hf = transformers.LlamaForCausalLM(hf_cfg).eval()
    lm = load_hf_llama(hf.state_dict(), hf_cfg, device="cuda", training=True)
    ids = torch.randint(0, 1024, (2, 150))
    with torch.no_grad():
        want = hf(ids).logits.reshape(-1, 1024)
    got = lm.forward_logits(ids.cuda()).reshape(300, -1)[:, :1024].float().cpu()
    torch.cuda.synchronize()
    _lib.check_status(torch.device("cuda", 0))
    assert (got - want).abs().max() < 0.05 * want.abs().max() + 0.02
    # one training step's loss against autograd through the independent implementation
    hf.train()
    out = hf(input_ids=ids, labels=ids)
    dev_ids = ids.cuda()
    lm.zero_grad()
    loss = lm.forward_loss(dev_ids[:, :-1].contiguous(), dev_ids[:, 1:].contiguous())
    lm.backward()
    torch.cuda.synchronize()
    _lib.check_status(torch.device("cuda", 0))
    assert abs(float(loss) - float(out.loss.detach())) < 0.03


def test_gpu_decoder_matches_transformers_gpt2():
    """LayerNorm, tanh-GELU, biases, a trained position table and the tied head on the bf16 kernel
    path against ``GPT2LMHeadModel`` in fp32."""
    transformers = pytest.importorskip("transformers")
    from coeus_b200.checkpoint.hf import load_hf_gpt2
    hf_cfg = transformers.GPT2Config(vocab_size=1024, n_positions=256, n_embd=256, n_layer=2,
                                     n_head=4, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    torch.manual_seed(0)
    hf = transformers.GPT2LMHeadModel(hf_cfg).eval()
    lm = load_hf_gpt2(hf.state_dict(), hf_cfg, device="cuda", training=True)
    ids = torch.randint(0, 1024, (2, 150))
    with torch.no_grad():
        want = hf(ids).logits.reshape(-1, 1024)
    got = lm.forward_logits(ids.cuda()).reshape(300, -1)[:, :1024].float().cpu()
    torch.cuda.synchronize()
    _lib.check_status(torch.device("cuda", 0))
    assert (got - want).abs().max() < 0.05 * want.abs().max() + 0.02
    hf.train()
    out = hf(input_ids=ids, labels=ids)
    out.loss.backward()
    dev_ids = ids.cuda()
    lm.zero_grad()
    loss = lm.forward_loss(dev_ids[:, :-1].contiguous(), dev_ids[:, 1:].contiguous())
    lm.backward()
    torch.cuda.synchronize()
    _lib.check_status(torch.device("cuda", 0))
    assert abs(float(loss) - float(out.loss.detach())) < 0.03
    g_want = hf.transformer.wpe.weight.grad
    g_got = lm.g["pos_embed"].float().cpu()
    assert (g_got - g_want).abs().max() <= 0.05 * g_want.abs().max() + 1e-4
