"""Mixture-of-experts layer on CPU: forward/backward against a dense PyTorch autograd restatement
(loop over experts with the same routing), single rank and expert-parallel over two Gloo ranks."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from coeus_b200.ops import moe as M
from coeus_b200.parallel.ep import ExpertParallel, MoEFFN, capacity_for

H, I, E, K, T = 32, 48, 4, 2, 40


def _reference(x, router, gate_up, down, resid, dout, aux_coef, cf):
    """Autograd restatement; ``gate_up [E,H,2I]``, ``down [E,I,H]``."""
    x = x.clone().requires_grad_(True)
    params = [p.clone().requires_grad_(True) for p in (router, gate_up, down)]
    r, gu_w, dn_w = params
    logits = x @ r
    probs = torch.softmax(logits, -1)
    C = capacity_for(T, E, K, cf)
    expert, w_, _, slot, _ = M.route(logits.detach(), K, C)
    pk = probs.gather(1, expert.long())
    w = pk / pk.sum(-1, keepdim=True)
    out = resid.clone()
    for k in range(K):
        for e in range(E):
            sel = (expert[:, k] == e) & (slot[:, k] >= 0)
            if sel.any():
                gu = x[sel] @ gu_w[e]
                act = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
                out = out.index_add(0, sel.nonzero()[:, 0], (act @ dn_w[e]) * w[sel, k][:, None])
    frac = torch.zeros(E).index_add_(0, expert.reshape(-1).long(), torch.ones(T * K)) / (T * K)
    aux = aux_coef * E * (frac * probs.mean(0)).sum()
    ((out * dout).sum() + aux).backward()
    return out.detach(), x.grad, [p.grad for p in params]


def _layer(epx, seed=3):
    m = MoEFFN(H, I, E, K, 1.25, epx, aux_coef=0.01, seed=seed, dtype=torch.float32)
    return m


def test_single_rank_matches_autograd():
    torch.manual_seed(0)
    epx = ExpertParallel(None, "cpu")
    m = _layer(epx)
    x, resid, dout = torch.randn(T, H), torch.randn(T, H), torch.randn(T, H)
    out = m.forward(x, resid)
    dx = m.backward(dout)
    ro, rdx, (gr, ggu, gdn) = _reference(x, m.master["router"], m.master["gate_up"],
                                         m.master["down"], resid, dout, 0.01, 1.25)
    assert (out - ro).abs().max() < 1e-5
    assert (dx - rdx).abs().max() < 1e-5
    assert (m.g["router"] - gr).abs().max() < 1e-5
    assert (m.g["gate_up"] - ggu).abs().max() < 1e-5
    assert (m.g["down"] - gdn).abs().max() < 1e-5


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, full, xs, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    epx = ExpertParallel(dist.group.WORLD, "cpu")
    m = _layer(epx)
    El = E // world
    m.master["router"].copy_(full["router"])
    m.master["gate_up"].copy_(full["gate_up"][rank * El:(rank + 1) * El])
    m.master["down"].copy_(full["down"][rank * El:(rank + 1) * El])
    m.sync_working_copy()
    x, resid, dout = (t[rank] for t in xs)
    o = m.forward(x, resid)
    dx = m.backward(dout)
    out.put((rank, o.numpy().copy(), dx.numpy().copy(), {k: v.numpy().copy() for k, v in m.g.items()}))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_expert_parallel_matches_autograd():
    torch.manual_seed(1)
    full = {"router": torch.randn(H, E) * 0.1, "gate_up": torch.randn(E, H, 2 * I) * 0.1,
            "down": torch.randn(E, I, H) * 0.1}
    xs = [torch.randn(2, T, H) for _ in range(3)]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, full, xs, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = {r[0]: r for r in (q.get(timeout=300) for _ in range(2))}
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    ggu = torch.zeros(E, H, 2 * I)
    gdn = torch.zeros(E, I, H)
    for rank in range(2):
        ro, rdx, (gr, g1, g2) = _reference(xs[0][rank], full["router"], full["gate_up"], full["down"],
                                           xs[1][rank], xs[2][rank], 0.01, 1.25)
        _, o, dx, g = res[rank]
        assert abs(torch.from_numpy(o) - ro).max() < 1e-5
        assert abs(torch.from_numpy(dx) - rdx).max() < 1e-5
        assert abs(torch.from_numpy(g["router"]) - gr).max() < 1e-5   # router grads are per rank
        ggu += g1
        gdn += g2
    El = E // 2
    for rank in range(2):   # expert gradients collect the tokens of both source ranks
        g = res[rank][3]
        assert abs(torch.from_numpy(g["gate_up"]) - ggu[rank * El:(rank + 1) * El]).max() < 1e-5
        assert abs(torch.from_numpy(g["down"]) - gdn[rank * El:(rank + 1) * El]).max() < 1e-5


# ---------------------------------------------------------------------------- whole model
def _moe_cfg():
    from coeus_b200.models.config import DecoderConfig
    return DecoderConfig(hidden_dim=32, num_layers=2, num_heads=2, intermediate_dim=48,
                         vocab_size=96, max_seq_len=16, use_bias=False, activation="swiglu",
                         norm="rmsnorm", pos="rope", num_experts=4, top_k=2, capacity_factor=2.0)


def test_moe_decoder_gradients_by_finite_differences():
    from coeus_b200.models.decoder import DecoderLM
    torch.manual_seed(0)
    m = DecoderLM(_moe_cfg(), device="cpu", dtype=torch.float32, seed=1)
    ids = torch.randint(0, 96, (2, 16))
    tgt = torch.randint(0, 96, (2, 16))
    m.zero_grad()
    m.forward_loss(ids, tgt)
    m.backward()
    for name in ("layers.0.moe.router_weights", "layers.1.moe.experts.gate_up_weights",
                 "layers.0.moe.experts.gate_up_weights", "layers.0.moe.experts.down_weights", "layers.0.attn.qkv_weights"):
        # directional derivative along the gradient: (L(w + e d) - L(w - e d)) / 2e = |g|
        w, g = m.master[name], m.g[name].clone()
        d = g / g.norm()
        eps = 3e-3   # small enough that no token changes its experts
        keep = w.clone()
        w.copy_(keep + eps * d); m.sync_working_copy(); lp = float(m.forward_loss(ids, tgt))
        w.copy_(keep - eps * d); m.sync_working_copy(); lm = float(m.forward_loss(ids, tgt))
        w.copy_(keep); m.sync_working_copy()
        fd = (lp - lm) / (2 * eps)
        assert abs(fd - float(g.norm())) < 4e-2 * float(g.norm()), (name, fd, float(g.norm()))


def _train_cfg():
    # eps = 1 keeps Adam from amplifying rounding noise of near-zero gradients into full steps
    from coeus_b200.train.trainer import TrainConfig
    return TrainConfig(learning_rate=0.05, eps=1.0, weight_decay=0.0)


def _train_worker(rank, world, port, ids, tgt, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.parallel.ep import ExpertParallelTrainer
    cfg = _moe_cfg()
    cfg.aux_loss_coef = 0.0
    m = DecoderLM(cfg, device="cpu", dtype=torch.float32, seed=1,
                  epx=ExpertParallel(dist.group.WORLD, "cpu"))
    tr = ExpertParallelTrainer(m, _train_cfg())
    losses = [float(tr.train_step(ids[rank], tgt[rank])) for _ in range(2)]
    out.put((rank, losses, {k: v.numpy().copy() for k, v in m.master.items()}))
    dist.barrier()
    dist.destroy_process_group()


def test_expert_parallel_training_matches_single_rank():
    """Two ranks with two experts each and half of the batch each == one rank with everything
    (capacity is ample, so no token is dropped on either side)."""
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.parallel.ep import ExpertParallelTrainer
    torch.manual_seed(2)
    ids = torch.randint(0, 96, (2, 2, 16))
    tgt = torch.randint(0, 96, (2, 2, 16))
    cfg = _moe_cfg()
    cfg.aux_loss_coef = 0.0
    single = DecoderLM(cfg, device="cpu", dtype=torch.float32, seed=1)
    tr = ExpertParallelTrainer(single, _train_cfg())
    ref_losses = [float(tr.train_step(ids.view(4, 16), tgt.view(4, 16))) for _ in range(2)]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_train_worker, args=(r, 2, port, ids, tgt, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = {r[0]: r for r in (q.get(timeout=300) for _ in range(2))}
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for step in range(2):
        mean = 0.5 * (res[0][1][step] + res[1][1][step])
        assert abs(mean - ref_losses[step]) < 1e-4
    for rank in range(2):
        for name, ref in single.master.items():
            got = torch.from_numpy(res[rank][2][name])
            if ".experts." in name:
                ref = ref[rank * 2:(rank + 1) * 2]
            assert (got - ref).abs().max() < 1e-5, name


def _worker_ep_ckpt(rank, world, port, tmp, out):
    import os
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.parallel.ep import ExpertParallel, ExpertParallelTrainer
    from coeus_b200.train.trainer import TrainConfig
    cfg = DecoderConfig(hidden_dim=32, num_layers=2, num_heads=2, intermediate_dim=48,
                        vocab_size=96, max_seq_len=16, use_bias=False, activation="swiglu",
                        norm="rmsnorm", pos="rope", num_experts=4, top_k=2, capacity_factor=2.0)
    epx = ExpertParallel(dist.group.WORLD, "cpu")
    tr = ExpertParallelTrainer(DecoderLM(cfg, "cpu", seed=2, dtype=torch.float32, epx=epx),
                               TrainConfig(learning_rate=0.05, eps=1.0, weight_decay=0.0,
                                           grad_clip=1e9))
    g = torch.Generator().manual_seed(rank)
    ids = torch.randint(0, 96, (2, 16), generator=g)
    tgt = torch.randint(0, 96, (2, 16), generator=g)
    for _ in range(2):
        tr.train_step(ids, tgt)
    # the norm the optimizer clipped by is the norm of all gradients of all ranks: expert
    # gradients live on one rank each, the rest is identical everywhere
    m = tr.model
    experts = torch.zeros(1)
    dense = torch.zeros(1)
    for sp in m.layout.specs:
        sq = (m.g32[sp.offset:sp.offset + sp.numel].double() ** 2).sum().float()
        if sp.expert:
            experts += sq
        else:
            dense += sq
    dist.all_reduce(experts)
    assert abs(float(tr.opt.grad_norm) - float(torch.sqrt(experts + dense))) < 1e-4 * float(tr.opt.grad_norm)
    tr.save_checkpoint(tmp)
    out.put((rank, {k: v.numpy().copy() for k, v in tr.model.master.items()}))
    dist.barrier()
    dist.destroy_process_group()


def test_expert_parallel_checkpoint_loads_into_one_rank(tmp_path):
    """Saved by two expert-parallel ranks (two experts each), loaded by a single rank holding all
    four: replicated tensors equal either rank's, expert rows are the ranks' rows in order."""
    import torch
    from mp_util import run_ranks
    from coeus_b200.checkpoint.named import load_named, model_state
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.optim.adamw import AdamW, AdamWConfig
    res = {r[0]: r[1] for r in run_ranks(_worker_ep_ckpt, 2, (str(tmp_path),), results=2)}
    cfg = DecoderConfig(hidden_dim=32, num_layers=2, num_heads=2, intermediate_dim=48,
                        vocab_size=96, max_seq_len=16, use_bias=False, activation="swiglu",
                        norm="rmsnorm", pos="rope", num_experts=4, top_k=2, capacity_factor=2.0)
    one = DecoderLM(cfg, "cpu", seed=7, dtype=torch.float32)
    opt = AdamW(AdamWConfig(), 0, one.n_flat, one.layout.decay_end, "cpu")
    man = load_named(str(tmp_path), model_state(one, opt))
    assert man["ep"] == 2 and man["opt_step"] == 2
    for name, t in one.master.items():
        spec = one.layout.by_name[name]
        if spec.expert:
            want = torch.cat([torch.from_numpy(res[0][name]), torch.from_numpy(res[1][name])], 0)
        else:
            want = torch.from_numpy(res[0][name])
        assert torch.equal(t, want), name
    assert float(opt.v.abs().sum()) > 0


def test_routing_stats_report_load_and_drops():
    import torch
    from coeus_b200.parallel.ep import ExpertParallel, MoEFFN
    torch.manual_seed(0)
    epx = ExpertParallel(None, "cpu")
    layer = MoEFFN(32, 48, 4, 2, 0.5, epx, dtype=torch.float32)      # capacity well below demand
    x = torch.randn(256, 32)
    layer.forward(x, torch.zeros_like(x), save=False)
    st = layer.routing_stats()
    assert abs(sum(st["load"]) - 1.0) < 1e-5 and st["max_over_mean"] >= 1.0
    assert 0.0 < st["dropped"] < 1.0
    roomy = MoEFFN(32, 48, 4, 2, 8.0, epx, dtype=torch.float32)
    roomy.forward(x, torch.zeros_like(x), save=False)
    assert roomy.routing_stats()["dropped"] == 0.0
