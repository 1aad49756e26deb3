"""The hand-written forward/backward of the decoder against PyTorch autograd on the same bf16
parameters, and a short training run."""
import pytest
import torch

from coeus_b200.models import torch_reference as R
from coeus_b200.models.config import DecoderConfig
from coeus_b200.models.decoder import DecoderLM
from coeus_b200.ops import _lib
from coeus_b200.train.trainer import TrainConfig, Trainer

pytestmark = pytest.mark.gpu

CFGS = {
    "gpt": DecoderConfig(hidden_dim=256, num_layers=2, num_heads=4, intermediate_dim=1024,
                         vocab_size=2048, max_seq_len=256),
    "llama": DecoderConfig(hidden_dim=256, num_layers=2, num_heads=2, intermediate_dim=512,
                           vocab_size=2048, max_seq_len=256, use_bias=False, activation="swiglu",
                           norm="rmsnorm", pos="rope"),
}


@pytest.mark.parametrize("kind", ["gpt", "llama"])
def test_forward_backward_matches_autograd(kind):
    cfg = CFGS[kind]
    torch.manual_seed(0)
    m = DecoderLM(cfg, device="cuda")
    for s in m.layout.specs:
        if s.kind in ("bias", "scale"):
            m.master[s.name].normal_(0.5 if s.kind == "scale" else 0.0, 0.2)
    m.sync_working_copy()
    batch = torch.randint(0, cfg.vocab_size, (3, 201), device="cuda")
    x, y = batch[:, :-1].contiguous(), batch[:, 1:].contiguous()
    m.zero_grad()
    loss = m.forward_loss(x, y)
    m.backward()
    torch.cuda.synchronize()
    _lib.check_status(torch.device("cuda", 0))
    params = {n: m.w[n].float().clone().requires_grad_(True) for n, _ in m.named_parameters()}
    ref = R.forward_loss(params, cfg, x, y)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 0.02
    for n in params:
        got, want = m.g[n], params[n].grad
        err = (got - want).abs().max().item()
        tol = 0.05 * want.abs().max().item() + 1e-4
        assert err <= tol, (n, err, tol)


def test_dropout_on_the_kernel_path_matches_the_host_path():
    """The same model, seed and step on the GPU (dropout in the GEMM epilogues, mask recomputed
    by the kernel in the backward pass, materialised attention-dropout path) and on the CPU
    restatement: equal masks, so loss and gradients agree to bf16 accuracy."""
    import dataclasses
    cfg = dataclasses.replace(CFGS["gpt"], dropout=0.2, attention_dropout=0.1)
    dev_m = DecoderLM(cfg, device="cuda", seed=5)
    cpu_m = DecoderLM(cfg, device="cpu", seed=5, dtype=torch.float32)
    cpu_m.p32.copy_(dev_m.p16.float().cpu())      # the host model computes on the bf16 weights
    cpu_m.sync_working_copy()
    batch = torch.randint(0, cfg.vocab_size, (2, 129), device="cuda")
    x, y = batch[:, :-1].contiguous(), batch[:, 1:].contiguous()
    for m, xx, yy in ((dev_m, x, y), (cpu_m, x.cpu(), y.cpu())):
        m.zero_grad()
        m.loss_value = float(m.forward_loss(xx, yy))
        m.backward()
    torch.cuda.synchronize()
    _lib.check_status(torch.device("cuda", 0))
    assert abs(dev_m.loss_value - cpu_m.loss_value) < 0.03
    for n, _ in dev_m.named_parameters():
        got, want = dev_m.g[n].cpu(), cpu_m.g[n]
        err = (got - want).abs().max().item()
        assert err <= 0.06 * want.abs().max().item() + 2e-4, (n, err)


@pytest.mark.parametrize("tie", [False, True])
def test_lm_head_in_vocabulary_slices_matches_the_whole_head(tie):
    """``lm_head_chunks``: loss and every gradient as with the logits held at once."""
    cfg = DecoderConfig(hidden_dim=256, num_layers=1, num_heads=4, intermediate_dim=512,
                        vocab_size=5000, max_seq_len=128, tie_embeddings=tie)
    torch.manual_seed(4)
    batch = torch.randint(0, cfg.vocab_size, (4, 101), device="cuda")
    x, y = batch[:, :-1].contiguous(), batch[:, 1:].contiguous()
    y[1, 5] = -100
    got = []
    for chunks in (1, 3):
        m = DecoderLM(cfg, device="cuda", seed=2, lm_head_chunks=chunks)
        m.zero_grad()
        loss = m.forward_loss(x, y)
        m.backward()
        torch.cuda.synchronize()
        _lib.check_status(torch.device("cuda", 0))
        got.append((float(loss), m.g32.clone()))
    assert len(m._head_chunks()) > 1
    assert abs(got[0][0] - got[1][0]) < 2e-3
    ref = got[0][1]
    assert (got[1][1] - ref).abs().max() < 0.02 * ref.abs().max() + 1e-4


def test_training_reduces_loss():
    cfg = CFGS["gpt"]
    m = DecoderLM(cfg, device="cuda")
    tr = Trainer(m, TrainConfig(learning_rate=1e-3))
    batch = torch.randint(0, cfg.vocab_size, (4, 129), device="cuda")
    losses = [float(tr.train_step(batch[:, :-1], batch[:, 1:])) for _ in range(8)]
    _lib.check_status(torch.device("cuda", 0))
    assert losses[-1] < losses[0] - 0.5, losses


def test_logits_last_only_matches_full():
    cfg = CFGS["gpt"]
    m = DecoderLM(cfg, device="cuda", training=False)
    ids = torch.randint(0, cfg.vocab_size, (2, 100), device="cuda")
    full = m.forward_logits(ids)
    last = m.forward_logits(ids, last_only=True)
    assert (full[:, -1].float() - last.float()).abs().max() < 0.05


@pytest.mark.parametrize("kind", ["gpt", "llama"])
def test_recompute_and_accumulation_match_the_plain_step(kind):
    """Activation recomputation reproduces the gradients; two accumulated micro-batches equal one
    step on their union (up to the order of fp32 sums)."""
    cfg = CFGS[kind]
    torch.manual_seed(1)
    batch = torch.randint(0, cfg.vocab_size, (4, 129), device="cuda")
    x, y = batch[:, :-1].contiguous(), batch[:, 1:].contiguous()
    grads = []
    for rc in (False, True):
        m = DecoderLM(cfg, device="cuda", seed=5, recompute=rc)
        m.zero_grad()
        m.forward_loss(x, y)
        m.backward()
        grads.append(m.g32.clone())
    scale = grads[0].abs().max()
    assert (grads[0] - grads[1]).abs().max() <= 2e-3 * scale
    a = Trainer(DecoderLM(cfg, device="cuda", seed=5), TrainConfig(learning_rate=1e-3, eps=1e-3))
    b = Trainer(DecoderLM(cfg, device="cuda", seed=5),
                TrainConfig(learning_rate=1e-3, eps=1e-3, grad_accum=2))
    a.train_step(x, y)
    b.train_step(x[:2].contiguous(), y[:2].contiguous())
    b.train_step(x[2:].contiguous(), y[2:].contiguous())
    torch.cuda.synchronize()
    _lib.check_status(torch.device("cuda", 0))
    assert b.step_index == 1
    d = (a.model.p32 - b.model.p32).abs()
    assert (d > 2e-4).float().mean() < 0.01


def test_fused_data_parallel_step_with_clipping_on_one_rank():
    """The split bucket kernel (modes 1 and 2) on a group of one rank against the plain trainer
    with the same clip threshold."""
    import os
    import torch.distributed as dist
    from mp_util import free_port
    from coeus_b200.parallel.zero import ShardedDataParallel
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(free_port())
    dev = torch.device("cuda", 0)
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    try:
        cfg = CFGS["gpt"]
        torch.manual_seed(2)
        batch = torch.randint(0, cfg.vocab_size, (2, 129), device="cuda")
        x, y = batch[:, :-1].contiguous(), batch[:, 1:].contiguous()
        tc = TrainConfig(learning_rate=1e-3, grad_clip=0.05)
        plain = Trainer(DecoderLM(cfg, device="cuda", seed=3), tc)
        dp = ShardedDataParallel(dist.group.WORLD, dev, backend="p2p")
        fused = Trainer(DecoderLM(cfg, device="cuda", seed=3), tc, dp=dp)
        for _ in range(3):
            la, lb = plain.train_step(x, y), fused.train_step(x, y)
        full = dp.gather_master()
        torch.cuda.synchronize()
        _lib.check_status(dev)
        assert abs(float(la) - float(lb)) < 0.02
        assert float(dp.grad_norm) > 0.05            # the threshold was active
        d = (plain.model.p32 - full).abs()
        assert (d > 5e-4).float().mean() < 0.01, d.max()
    finally:
        dist.destroy_process_group()
