"""Tensor-parallel decoder on CPU ranks (Gloo, tp = 2): loss and gradients equal the unsharded
model's, shard by shard."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from coeus_b200.models.config import DecoderConfig
from coeus_b200.models.decoder import DecoderLM

CFG = DecoderConfig(hidden_dim=64, num_layers=2, num_heads=4, intermediate_dim=96,
                    vocab_size=250, max_seq_len=32, use_bias=False, activation="swiglu",
                    norm="rmsnorm", pos="rope")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker_ckpt(rank, world, port, batch, tmp, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from coeus_b200.checkpoint.formats import load_model
    from coeus_b200.optim.adamw import AdamWConfig
    from coeus_b200.parallel.tp import TensorParallel
    from coeus_b200.parallel.tp_model import TPDecoderLM, TPTrainer
    tp = TensorParallel(dist.group.WORLD, "cpu")
    x, y = batch[:, :-1].contiguous(), batch[:, 1:].contiguous()
    oc = AdamWConfig(lr=1e-2)
    a = TPTrainer(TPDecoderLM(CFG, tp, "cpu", dtype=torch.float32, seed=0), oc)
    for _ in range(2):
        a.train_step(x, y)
    a.save_checkpoint(tmp + "/ckpt")
    a.model.save(tmp + "/full.safetensors")
    # resume into a differently initialised trainer: the next step is the same step
    b = TPTrainer(TPDecoderLM(CFG, tp, "cpu", dtype=torch.float32, seed=9), AdamWConfig(lr=1e-2))
    man = b.load_checkpoint(tmp + "/ckpt")
    assert man["train_step"] == 2 and torch.equal(a.model.p32, b.model.p32)
    la, lb = float(a.train_step(x, y)), float(b.train_step(x, y))
    assert la == lb and torch.equal(a.model.p32, b.model.p32)
    # the exported whole model gives the loss the shards gave before that step
    full, _ = load_model(tmp + "/full.safetensors", device="cpu")
    c = TPDecoderLM(CFG, tp, "cpu", dtype=torch.float32, full=full)
    b2 = TPTrainer(TPDecoderLM(CFG, tp, "cpu", dtype=torch.float32, seed=9), AdamWConfig(lr=1e-2))
    b2.load_checkpoint(tmp + "/ckpt")
    assert torch.equal(c.p32, b2.model.p32)
    out.put((rank, la, float(full.forward_loss(x, y))))
    dist.barrier()
    dist.destroy_process_group()


def test_tp_checkpoint_resume_and_whole_model_export(tmp_path):
    from mp_util import run_ranks
    torch.manual_seed(0)
    batch = torch.randint(0, CFG.vocab_size, (2, 17))
    res = run_ranks(_worker_ckpt, 2, (batch, str(tmp_path)), results=2)
    ref = DecoderLM(CFG, device="cpu", seed=0, dtype=torch.float32)
    from coeus_b200.optim.adamw import AdamW, AdamWConfig
    opt = AdamW(AdamWConfig(lr=1e-2), 0, ref.n_flat, ref.layout.decay_end, "cpu")
    x, y = batch[:, :-1].contiguous(), batch[:, 1:].contiguous()
    for _ in range(2):
        ref.zero_grad()
        ref.forward_loss(x, y)
        ref.backward()
        opt.step(ref.p32, ref.g32, ref.p16)
    want = float(ref.forward_loss(x, y))
    for _, la, lfull in res:
        assert abs(la - want) < 1e-4 and abs(lfull - want) < 1e-4


def _worker(rank, world, port, batch, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from coeus_b200.parallel.tp import TensorParallel
    from coeus_b200.parallel.tp_model import TPDecoderLM
    full = DecoderLM(CFG, device="cpu", seed=0, dtype=torch.float32)
    tp = TensorParallel(dist.group.WORLD, "cpu")
    m = TPDecoderLM(CFG, tp, "cpu", dtype=torch.float32, full=full)
    # the seed-based init draws what the unsharded model with that seed holds at this rank's place
    seeded = TPDecoderLM(CFG, tp, "cpu", dtype=torch.float32, seed=0)
    assert torch.equal(seeded.p32, m.p32)
    x, y = batch[:, :-1].contiguous(), batch[:, 1:].contiguous()
    m.zero_grad()
    loss = m.forward_loss(x, y)
    m.backward()
    # activation recomputation must reproduce the same gradients bit for bit
    m2 = TPDecoderLM(CFG, tp, "cpu", dtype=torch.float32, full=full, recompute=True)
    m2.zero_grad()
    loss2 = m2.forward_loss(x, y)
    assert all(set(a) == {"x"} for a in m2._saved["layers"])
    m2.backward()
    assert float(loss2) == float(loss) and torch.equal(m2.g32, m.g32)
    out.put((rank, float(loss), {k: v.numpy().copy() for k, v in m.g.items()}))
    dist.barrier()
    dist.destroy_process_group()


def test_tp2_matches_unsharded():
    torch.manual_seed(0)
    batch = torch.randint(0, CFG.vocab_size, (2, 17))
    x, y = batch[:, :-1].contiguous(), batch[:, 1:].contiguous()
    full = DecoderLM(CFG, device="cpu", seed=0, dtype=torch.float32)
    full.zero_grad()
    ref_loss = float(full.forward_loss(x, y))
    full.backward()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, batch, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    H, I = CFG.hidden_dim, CFG.intermediate_dim
    Hl, Il, Vl = H // 2, I // 2, CFG.vocab_padded // 2
    for rank, loss, g in results:
        g = {k: torch.from_numpy(v) for k, v in g.items()}
        assert abs(loss - ref_loss) < 1e-4
        fg = full.g
        assert (g["token_embed"] - fg["token_embed"]).abs().max() < 1e-5
        assert (g["output_proj"] - fg["output_proj"][:, rank * Vl:(rank + 1) * Vl]).abs().max() < 1e-5
        for l in range(CFG.num_layers):
            p = f"layers.{l}."
            want = torch.cat([fg[p + "attn.qkv_weights"][:, i * H + rank * Hl:i * H + (rank + 1) * Hl]
                              for i in range(3)], 1)
            assert (g[p + "attn.qkv_weights"] - want).abs().max() < 1e-5
            assert (g[p + "attn.o_weights"] - fg[p + "attn.o_weights"][rank * Hl:(rank + 1) * Hl]).abs().max() < 1e-5
            wg = fg[p + "ff.gate_up_weights"]
            want = torch.cat([wg[:, rank * Il:(rank + 1) * Il], wg[:, I + rank * Il:I + (rank + 1) * Il]], 1)
            assert (g[p + "ff.up_weights"] - want).abs().max() < 1e-5
            assert (g[p + "ff.down_weights"] - fg[p + "ff.down_weights"][rank * Il:(rank + 1) * Il]).abs().max() < 1e-5
            assert (g[p + "norm1_scale"] - fg[p + "norm1_scale"]).abs().max() < 1e-5
            assert (g[p + "norm2_scale"] - fg[p + "norm2_scale"]).abs().max() < 1e-5
        assert (g["final_norm_scale"] - fg["final_norm_scale"]).abs().max() < 1e-5


GQA = DecoderConfig(hidden_dim=64, num_layers=2, num_heads=8, num_kv_heads=4, intermediate_dim=96,
                    vocab_size=250, max_seq_len=32, use_bias=False, activation="swiglu",
                    norm="rmsnorm", pos="rope", rope_llama3=(8.0, 1.0, 4.0, 8))


def _worker_gqa(rank, world, port, batch, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from coeus_b200.infer.tp_engine import TPInferenceEngine
    from coeus_b200.parallel.tp import TensorParallel
    from coeus_b200.parallel.tp_model import TPDecoderLM
    full = DecoderLM(GQA, device="cpu", seed=0, dtype=torch.float32)
    tp = TensorParallel(dist.group.WORLD, "cpu")
    m = TPDecoderLM(GQA, tp, "cpu", dtype=torch.float32, full=full)
    x, y = batch[:, :-1].contiguous(), batch[:, 1:].contiguous()
    m.zero_grad()
    loss = m.forward_loss(x, y)
    m.backward()
    whole = m.gather_full()        # shards put back together = the model they were cut from
    same = all(torch.equal(whole[k], full.master[k]) for k in
               ("layers.0.attn.qkv_weights", "layers.1.attn.o_weights", "output_proj"))
    toks = TPInferenceEngine(m, max_batch=2).generate(x[:, :8].contiguous(), 5)
    out.put((rank, float(loss), same, toks.numpy().copy(),
             {k: v.numpy().copy() for k, v in m.g.items() if "attn" in k}))
    dist.barrier()
    dist.destroy_process_group()


def test_tp2_grouped_query_attention_matches_unsharded():
    """Llama-3.1 style model (grouped-query attention, scaled rotary frequencies).  Every rank
    holds whole groups (4 query heads with their 2 K/V heads): loss, the narrow
    fused-QKV gradient shard, the reassembled weights and generation equal the unsharded model."""
    from coeus_b200.infer.engine import InferenceEngine
    torch.manual_seed(0)
    batch = torch.randint(0, GQA.vocab_size, (2, 17))
    x, y = batch[:, :-1].contiguous(), batch[:, 1:].contiguous()
    full = DecoderLM(GQA, device="cpu", seed=0, dtype=torch.float32)
    full.zero_grad()
    ref_loss = float(full.forward_loss(x, y))
    full.backward()
    want_toks = InferenceEngine(full, max_batch=2).generate(x[:, :8].contiguous(), 5)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_gqa, args=(r, 2, port, batch, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    H, Hkv = GQA.hidden_dim, GQA.kv_dim
    Hl, Kl = H // 2, Hkv // 2
    for rank, loss, same, toks, g in results:
        assert same and abs(loss - ref_loss) < 1e-4
        assert torch.equal(torch.from_numpy(toks), want_toks)
        for l in range(GQA.num_layers):
            p = f"layers.{l}."
            fg = full.g[p + "attn.qkv_weights"]
            want = torch.cat([fg[:, rank * Hl:(rank + 1) * Hl],
                              fg[:, H + rank * Kl:H + (rank + 1) * Kl],
                              fg[:, H + Hkv + rank * Kl:H + Hkv + (rank + 1) * Kl]], 1)
            assert (torch.from_numpy(g[p + "attn.qkv_weights"]) - want).abs().max() < 1e-5
