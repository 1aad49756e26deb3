"""Tensor-parallel generation on two Gloo ranks against the single-rank engine."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _cfg():
    from coeus_b200.models.config import DecoderConfig
    return DecoderConfig(hidden_dim=32, num_layers=2, num_heads=4, intermediate_dim=48,
                         vocab_size=96, max_seq_len=64, use_bias=False, activation="swiglu",
                         norm="rmsnorm", pos="rope")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ids, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from coeus_b200.infer.tp_engine import TPInferenceEngine
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.parallel.tp import TensorParallel
    from coeus_b200.parallel.tp_model import TPDecoderLM
    full = DecoderLM(_cfg(), "cpu", seed=5, dtype=torch.float32, training=False)
    tp = TensorParallel(dist.group.WORLD, "cpu", backend="nccl")
    m = TPDecoderLM(_cfg(), tp, "cpu", dtype=torch.float32, full=full)
    eng = TPInferenceEngine(m, max_batch=4)
    toks = eng.generate(ids, 6)
    out.put((rank, toks.numpy().copy()))
    dist.barrier()
    dist.destroy_process_group()


def test_tp_generation_matches_single_rank_engine():
    from coeus_b200.infer.engine import InferenceEngine
    from coeus_b200.models.decoder import DecoderLM
    torch.manual_seed(0)
    ids = torch.randint(0, 96, (4, 8))
    full = DecoderLM(_cfg(), "cpu", seed=5, dtype=torch.float32, training=False)
    want = InferenceEngine(full, max_batch=4).generate(ids, 6)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ids, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, toks in res:
        assert torch.equal(torch.from_numpy(toks), want), rank


def _worker_serving(rank, world, port, prompts, budgets, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from coeus_b200.infer.scheduler import ContinuousBatcher
    from coeus_b200.infer.tp_engine import TPInferenceEngine
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.parallel.tp import TensorParallel
    from coeus_b200.parallel.tp_model import TPDecoderLM
    full = DecoderLM(_cfg(), "cpu", seed=5, dtype=torch.float32, training=False)
    tp = TensorParallel(dist.group.WORLD, "cpu", backend="nccl")
    m = TPDecoderLM(_cfg(), tp, "cpu", dtype=torch.float32, full=full)
    # max_batch 2 < longest prompt: prompts take the library all-reduce, decode rows the
    # engine's all-reduce buffers
    cb = ContinuousBatcher(TPInferenceEngine(m, max_batch=2), max_seqs=2, max_len=64)
    ids = [cb.submit(p, k) for p, k in zip(prompts, budgets)]
    res = cb.run()
    out.put((rank, [res[i] for i in ids]))
    dist.barrier()
    dist.destroy_process_group()


def test_tp_continuous_batching_matches_single_rank_engine():
    """Requests of different lengths through the batcher on two tensor-parallel ranks: every rank
    produces the tokens the single-rank engine produces for each request alone."""
    from mp_util import run_ranks
    from coeus_b200.infer.engine import InferenceEngine
    from coeus_b200.models.decoder import DecoderLM
    torch.manual_seed(3)
    prompts = [torch.randint(0, 96, (n,)).tolist() for n in (5, 11, 3, 20)]
    budgets = [4, 6, 2, 5]
    full = DecoderLM(_cfg(), "cpu", seed=5, dtype=torch.float32, training=False)
    want = [InferenceEngine(full, max_batch=1).generate(torch.tensor(p)[None], k)[0, len(p):].tolist()
            for p, k in zip(prompts, budgets)]
    for rank, got in run_ranks(_worker_serving, 2, (prompts, budgets), results=2):
        assert got == want, rank


def _worker_tp_serving(rank, world, port, prompts, budgets, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from coeus_b200.infer.tp_engine import TPInferenceEngine
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.parallel.tp import TensorParallel
    from coeus_b200.parallel.tp_model import TPDecoderLM
    from coeus_b200.serve import ServingLoop
    full = DecoderLM(_cfg(), "cpu", seed=5, dtype=torch.float32, training=False)
    tp = TensorParallel(dist.group.WORLD, "cpu", backend="nccl")
    m = TPDecoderLM(_cfg(), tp, "cpu", dtype=torch.float32, full=full)
    loop = ServingLoop(None, max_seqs=2, max_len=64, engine=TPInferenceEngine(m, max_batch=2),
                       group=dist.group.WORLD)
    if rank == 0:                       # the leader takes the requests ...
        futs = [loop.submit(p, k) for p, k in zip(prompts, budgets)]
        res = [f.result(timeout=120) for f in futs]
        slow = loop.submit(prompts[0], 40)
        loop.cancel(slow)               # ... and cancellations and the stop reach the followers
        late = loop.submit(prompts[1], 2).result(timeout=120)
        loop.close()
        out.put((rank, res, late, loop.counters["completed"]))
    else:
        loop.join(timeout=200)          # followers step along until the leader stops the loop
        assert not loop.healthy()
        out.put((rank, None, None, 0))
    dist.barrier()
    dist.destroy_process_group()


def test_tp_serving_loop_leader_and_follower():
    from mp_util import run_ranks
    from coeus_b200.infer.engine import InferenceEngine
    from coeus_b200.models.decoder import DecoderLM
    torch.manual_seed(3)
    prompts = [torch.randint(0, 96, (n,)).tolist() for n in (5, 11, 3)]
    budgets = [4, 6, 2]
    full = DecoderLM(_cfg(), "cpu", seed=5, dtype=torch.float32, training=False)
    want = [InferenceEngine(full, max_batch=1).generate(torch.tensor(p)[None], k)[0, len(p):].tolist()
            for p, k in zip(prompts, budgets)]
    res = {r[0]: r for r in run_ranks(_worker_tp_serving, 2, (prompts, budgets), results=2)}
    assert res[0][1] == want and res[0][2] == want[1][:2] and res[0][3] == 4
