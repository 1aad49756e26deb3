"""Pipeline parallelism on two GPUs against one GPU with gradient accumulation: the 1F1B schedule
over NCCL point-to-point and over NVLink peer memory, and the interleaved schedule (two chunks of
blocks per rank) over peer memory."""
import os

import pytest
import torch
import torch.distributed as dist

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _cfg():
    from coeus_b200.models.config import DecoderConfig
    return DecoderConfig(hidden_dim=256, num_layers=4, num_heads=4, intermediate_dim=512,
                         vocab_size=512, max_seq_len=128, use_bias=False, activation="swiglu",
                         norm="rmsnorm", pos="rope")


def _train_cfg():
    from coeus_b200.train.trainer import TrainConfig
    return TrainConfig(learning_rate=0.05, eps=1.0, weight_decay=0.0)


def _worker(rank, world, port, ids, tgt, mode, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from coeus_b200.ops import _lib
    from coeus_b200.parallel.pp import InterleavedPipelineStage, PipelineStage
    mode, _, slots = mode.partition("-")
    slots = slots or "bounded"
    if mode == "interleaved":
        st = InterleavedPipelineStage(_cfg(), dist.group.WORLD, dev, micro_batches=ids.shape[0],
                                      chunks=2, seed=4, train_cfg=_train_cfg(),
                                      peer_wait_ms=5000.0, peer_slots=slots)
        assert st.transport == "peer"
        models = st.models
    else:
        st = PipelineStage(_cfg(), dist.group.WORLD, dev, micro_batches=ids.shape[0], seed=4,
                           train_cfg=_train_cfg(), transport=mode, peer_wait_ms=5000.0,
                           peer_slots=slots)
        models = [st.model]
    ids, tgt = ids.to(dev), tgt.to(dev)
    losses = [float(st.train_step(ids, tgt)) for _ in range(3)]
    torch.cuda.synchronize()
    _lib.check_status(dev)
    if getattr(st, "_ring", None) is not None:
        # bounded: a handful of slots however many micro-batches; message: one per message
        from coeus_b200.parallel.pp import ring_depths
        bounded = ring_depths(world, ids.shape[0], len(models))
        for kind in ("f", "b"):
            n = ids.shape[0] * len(models)
            assert st._ring.depths[kind] == (n if slots == "message" else bounded[kind])
            assert bounded[kind] <= 3 < n + 1
    weights = {k: v.float().cpu().numpy().copy() for m in models for k, v in m.master.items()}
    out.put((rank, losses, weights))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["nccl", "peer", "peer-message", "interleaved",
                                  "interleaved-message"])
def test_two_stage_pipeline_matches_one_gpu(mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from mp_util import run_ranks
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.optim.adamw import AdamW
    torch.manual_seed(0)
    M, b, S = 4, 2, 128
    ids = torch.randint(0, 512, (M, b, S))
    tgt = torch.randint(0, 512, (M, b, S))
    full = DecoderLM(_cfg(), "cuda", seed=4)
    opt = AdamW(_train_cfg().adamw(), 0, full.n_flat, full.layout.decay_end, "cuda")
    ref_losses = []
    for _ in range(3):
        full.zero_grad()
        tot = 0.0
        for i in range(M):
            tot += float(full.forward_loss(ids[i].cuda(), tgt[i].cuda(),
                                           grad_scale=1.0 / (b * S * M))) / M
            full.backward()
        opt.step(full.p32, full.g32, full.p16, 1.0)
        ref_losses.append(tot)
    res = {r[0]: r for r in run_ranks(_worker, 2, (ids, tgt, mode), results=2, timeout=150.0)}
    for step in range(3):
        assert abs(res[1][1][step] - ref_losses[step]) < 2e-2
    for rank in range(2):
        for name, got in res[rank][2].items():
            ref = full.master[name].float().cpu()
            got = torch.from_numpy(got)
            assert (got - ref).abs().max() < 5e-3 * max(1.0, float(ref.abs().max())), name
