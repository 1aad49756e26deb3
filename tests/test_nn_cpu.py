"""Autograd wrappers: gradients of every layer against plain PyTorch autograd on the same math
(CPU restatement of the kernels; the GPU kernels themselves are covered by the kernel tests)."""
import pytest
import torch

from coeus_b200 import nn as cnn
from coeus_b200.nn import functional as F


def _ref_attention(qkv, B, S, nh, dh):
    H = nh * dh
    q, k, v = (t.reshape(B, S, nh, dh).transpose(1, 2) for t in (qkv[:, :H], qkv[:, H:2 * H], qkv[:, 2 * H:]))
    o = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
    return o.transpose(1, 2).reshape(B * S, H)


def test_block_gradients_match_pytorch():
    torch.manual_seed(0)
    B, S, D, nh, I = 2, 8, 16, 2, 24
    blk = cnn.Block(D, nh, I, rms=False, bias=True, swiglu=False, rope=False, device="cpu")
    x = torch.randn(B * S, D, requires_grad=True)
    y = blk(x, B, S)
    y.square().sum().backward()
    got = {n: p.grad.clone() for n, p in blk.named_parameters()}
    gx = x.grad.clone()
    # the same block written with stock PyTorch ops
    x2 = x.detach().clone().requires_grad_(True)
    p = {n: t.detach().clone().requires_grad_(True) for n, t in blk.named_parameters()}
    ln = torch.nn.functional.layer_norm
    n1 = ln(x2, (D,), p["norm1.scale"], p["norm1.bias"], 1e-5)
    qkv = n1 @ p["attn.qkv.weight"] + p["attn.qkv.bias"]
    a = _ref_attention(qkv, B, S, nh, D // nh) @ p["attn.o.weight"] + p["attn.o.bias"]
    xm = x2 + a
    n2 = ln(xm, (D,), p["norm2.scale"], p["norm2.bias"], 1e-5)
    h = torch.nn.functional.gelu(n2 @ p["mlp.up.weight"] + p["mlp.up.bias"], approximate="tanh")
    out = xm + h @ p["mlp.down.weight"] + p["mlp.down.bias"]
    out.square().sum().backward()
    assert (y - out).abs().max() < 1e-4
    assert (gx - x2.grad).abs().max() < 1e-3
    for n in got:
        assert (got[n] - p[n].grad).abs().max() < 1e-3 * max(1.0, p[n].grad.abs().max()), n


def test_swiglu_rope_rms_embedding_and_loss():
    torch.manual_seed(1)
    B, S, D, nh, V = 2, 8, 16, 2, 40
    emb = cnn.Embedding(V, D, device="cpu")
    blk = cnn.Block(D, nh, 24, rms=True, bias=False, swiglu=True, rope=True, device="cpu")
    head = cnn.Linear(D, V, bias=False, device="cpu")
    with torch.no_grad():       # larger weights: gradients well above fp32 rounding of the loss
        for prm in list(blk.parameters()) + [head.weight, emb.weight]:
            if prm.dim() == 2:
                prm.mul_(10.0)
    ids = torch.randint(0, V, (B, S))
    tgt = torch.randint(0, V, (B, S))
    loss = cnn.CrossEntropyLoss()(head(blk(emb(ids), B, S)), tgt)
    loss.backward()
    # finite differences along the gradient of a few parameters
    for prm in (emb.weight, blk.attn.qkv.weight, blk.mlp.up.weight, blk.norm2.scale, head.weight):
        g = prm.grad.clone()
        d = g / g.norm()
        eps = 2e-3
        with torch.no_grad():
            prm.add_(eps * d); lp = float(cnn.CrossEntropyLoss()(head(blk(emb(ids), B, S)), tgt))
            prm.sub_(2 * eps * d); lm = float(cnn.CrossEntropyLoss()(head(blk(emb(ids), B, S)), tgt))
            prm.add_(eps * d)
        fd = (lp - lm) / (2 * eps)
        assert abs(fd - float(g.norm())) < 3e-2 * float(g.norm()) + 1e-5


def test_functional_softmax_and_gelu_values():
    # unit values the reference tests (plugins/model-transformer/src/lib.rs:1153-1192)
    s = F.softmax(torch.tensor([[1.0, 2.0, 3.0]]))
    assert abs(float(s.sum()) - 1.0) < 1e-6 and s[0, 2] > s[0, 1] > s[0, 0]
    assert abs(float(F.gelu(torch.tensor([[0.0]])))) < 1e-6
    assert float(F.gelu(torch.tensor([[1.0]]))) > 0 > float(F.gelu(torch.tensor([[-1.0]])))


@pytest.mark.parametrize("kind", ["gpt", "llama", "tied", "gqa"])
def test_autograd_transformer_matches_the_explicit_decoder(kind):
    """The nn.Module model with the explicit decoder's weights: same loss, and autograd's
    gradients equal the hand-written backward pass."""
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.nn import TransformerLM
    kw = dict(hidden_dim=32, num_layers=2, num_heads=2, intermediate_dim=64, vocab_size=64,
              max_seq_len=16)
    if kind in ("llama", "gqa"):
        kw.update(use_bias=False, activation="swiglu", norm="rmsnorm", pos="rope")
    if kind == "gqa":                  # 4 query heads reading 2 key/value heads
        kw.update(num_heads=4, num_kv_heads=2)
    if kind == "tied":
        kw.update(tie_embeddings=True)
    cfg = DecoderConfig(**kw)
    lm = DecoderLM(cfg, "cpu", seed=3, dtype=torch.float32)
    for s in lm.layout.specs:                       # non-trivial norm scales and biases
        if s.kind in ("bias", "scale"):
            lm.master[s.name].normal_(1.0 if s.kind == "scale" else 0.0, 0.1)
    lm.sync_working_copy()
    net = TransformerLM(cfg, device="cpu")
    net.load_from(lm)
    torch.manual_seed(0)
    ids = torch.randint(0, 64, (2, 16))
    tgt = torch.randint(0, 64, (2, 16))
    lm.zero_grad()
    want = lm.forward_loss(ids, tgt)
    lm.backward()
    loss = net(ids, tgt)
    loss.backward()
    assert abs(float(loss.detach()) - float(want)) < 1e-5
    blk = net.blocks[1]
    assert torch.allclose(blk.attn.qkv.weight.grad, lm.g["layers.1.attn.qkv_weights"], atol=1e-5)
    assert torch.allclose(blk.mlp.down.weight.grad, lm.g["layers.1.ff.down_weights"], atol=1e-5)
    assert torch.allclose(net.embed.weight.grad, lm.g["token_embed"][:64], atol=1e-5)
    n1 = lm.layout.norm_names[0]
    assert torch.allclose(net.blocks[0].norm1.scale.grad, lm.g[f"layers.0.{n1}_scale"], atol=1e-5)
    assert net(ids).shape == (32, 64)


def test_module_adamw_matches_torch_adamw():
    from coeus_b200.nn import Block
    from coeus_b200.optim.adamw import AdamWConfig
    from coeus_b200.optim.module import ModuleAdamW
    torch.manual_seed(0)
    a = Block(32, 2, 64, device="cpu")
    b = Block(32, 2, 64, device="cpu")
    b.load_state_dict(a.state_dict())
    decay = [p for n, p in b.named_parameters() if p.dim() >= 2]
    plain = [p for n, p in b.named_parameters() if p.dim() < 2]
    ref = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1},
                             {"params": plain, "weight_decay": 0.0}],
                            lr=1e-2, betas=(0.9, 0.95), eps=1e-3)
    # eps well above rounding noise: the key bias has a mathematically zero gradient, and Adam
    # with a tiny eps turns its rounding noise into full-size steps of random sign
    mine = ModuleAdamW(a, AdamWConfig(1e-2, 0.9, 0.95, 1e-3, 0.1, None))
    x = torch.randn(2 * 8, 32)
    for _ in range(4):
        for net, opt in ((a, mine), (b, ref)):
            opt.zero_grad()
            net(x, 2, 8).pow(2).mean().backward()
            opt.step()
    for (n, p), (_, q) in zip(a.named_parameters(), b.named_parameters()):
        assert torch.allclose(p, q, atol=2e-6), n
    # the parameters are views of one flat buffer
    assert all(p.data_ptr() >= mine.p16.data_ptr() for _, p, _ in mine.params)


def _worker_module_dp(rank, world, port, x, out):
    import os
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from coeus_b200.nn import Block
    from coeus_b200.optim.adamw import AdamWConfig
    from coeus_b200.optim.module import ModuleAdamW
    torch.manual_seed(100 + rank)                 # replicas start differently; rank 0 wins
    net = Block(32, 2, 64, device="cpu")
    opt = ModuleAdamW(net, AdamWConfig(1e-2, 0.9, 0.95, 1e-3, 0.1, None), group=dist.group.WORLD)
    mine = x[rank * 8:(rank + 1) * 8]             # one sequence of 8 tokens per rank
    for _ in range(3):
        opt.zero_grad()
        net(mine, 1, 8).pow(2).mean().backward()
        opt.step()
    out.put((rank, opt.p32.numpy().copy()))
    dist.barrier()
    dist.destroy_process_group()


def test_module_adamw_data_parallel_matches_one_process():
    import sys
    import os
    sys.path.insert(0, os.path.dirname(__file__))
    from mp_util import run_ranks
    from coeus_b200.nn import Block
    from coeus_b200.optim.adamw import AdamWConfig
    from coeus_b200.optim.module import ModuleAdamW
    torch.manual_seed(7)
    x = torch.randn(16, 32)
    res = {r[0]: torch.from_numpy(r[1]) for r in run_ranks(_worker_module_dp, 2, (x,), results=2)}
    assert torch.equal(res[0], res[1])            # replicas stay identical
    torch.manual_seed(100)                        # rank 0's initial weights
    net = Block(32, 2, 64, device="cpu")
    opt = ModuleAdamW(net, AdamWConfig(1e-2, 0.9, 0.95, 1e-3, 0.1, None))
    for _ in range(3):
        opt.zero_grad()
        # the mean over both ranks' sequences
        (0.5 * (net(x[:8], 1, 8).pow(2).mean() + net(x[8:], 1, 8).pow(2).mean())).backward()
        opt.step()
    assert torch.allclose(opt.p32, res[0], atol=2e-6)
