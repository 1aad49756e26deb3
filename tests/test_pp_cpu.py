"""Pipeline parallelism on CPU ranks (Gloo): the 1F1B schedule itself, and a two- and three-stage
training step against the same model on one rank with gradient accumulation."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from coeus_b200.parallel.pp import (comm_order, nccl_order_deadlocks, ring_depths, schedule_1f1b,
                                     schedule_interleaved, split_layers)


def test_split_layers():
    assert split_layers(5, 2) == [(0, 3), (3, 5)]
    assert split_layers(24, 8) == [(3 * i, 3 * i + 3) for i in range(8)]
    with pytest.raises(Exception):
        split_layers(2, 3)


@pytest.mark.parametrize("P,M", [(1, 3), (2, 4), (4, 8), (4, 2), (3, 3)])
def test_schedule_is_valid_1f1b(P, M):
    for s in range(P):
        steps = schedule_1f1b(s, P, M)
        assert sorted(i for k, i in steps if k == "F") == list(range(M))
        assert sorted(i for k, i in steps if k == "B") == list(range(M))
        alive, peak = set(), 0
        for k, i in steps:
            if k == "F":
                alive.add(i)
            else:
                assert i in alive       # a backward only after its forward
                alive.remove(i)
            peak = max(peak, len(alive))
        assert peak <= min(P - s, M)    # bounded activation stash


def _cfg(moe=False, pos="rope"):
    from coeus_b200.models.config import DecoderConfig
    kw = dict(num_experts=4, top_k=2, capacity_factor=2.0, aux_loss_coef=0.0) if moe else {}
    return DecoderConfig(hidden_dim=32, num_layers=3, num_heads=2, intermediate_dim=48,
                         vocab_size=96, max_seq_len=16, use_bias=False, activation="swiglu",
                         norm="rmsnorm", pos=pos, **kw)


def _train_cfg():
    from coeus_b200.train.trainer import TrainConfig
    return TrainConfig(learning_rate=0.05, eps=1.0, weight_decay=0.0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ids, tgt, out, pos="rope"):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from coeus_b200.parallel.pp import PipelineStage
    st = PipelineStage(_cfg(pos=pos), dist.group.WORLD, "cpu", micro_batches=ids.shape[0], seed=4,
                       dtype=torch.float32, train_cfg=_train_cfg())
    losses = [float(st.train_step(ids, tgt)) for _ in range(2)]
    out.put((rank, losses, {k: v.numpy().copy() for k, v in st.model.master.items()}))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_pipeline_training_matches_single_rank(world):
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.optim.adamw import AdamW
    torch.manual_seed(0)
    M, b, S = 4, 2, 16
    ids = torch.randint(0, 96, (M, b, S))
    tgt = torch.randint(0, 96, (M, b, S))
    # three stages run with a trained position table (its gradient is the first stage's)
    pos = "learned" if world == 3 else "rope"
    full = DecoderLM(_cfg(pos=pos), "cpu", seed=4, dtype=torch.float32)
    opt = AdamW(_train_cfg().adamw(), 0, full.n_flat, full.layout.decay_end, "cpu")
    ref_losses = []
    for _ in range(2):
        full.zero_grad()
        tot = 0.0
        for i in range(M):
            tot += float(full.forward_loss(ids[i], tgt[i], grad_scale=1.0 / (b * S * M))) / M
            full.backward()
        opt.step(full.p32, full.g32, full.p16, 1.0)
        ref_losses.append(tot)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ids, tgt, q, pos))
             for r in range(world)]
    for p in procs:
        p.start()
    res = {r[0]: r for r in (q.get(timeout=300) for _ in range(world))}
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for step in range(2):
        assert abs(res[world - 1][1][step] - ref_losses[step]) < 1e-5
    seen = set()
    for rank in range(world):
        for name, got in res[rank][2].items():
            assert (torch.from_numpy(got) - full.master[name]).abs().max() < 1e-5, name
            seen.add(name)
    assert seen == set(full.master)     # every tensor lives on exactly the stages that need it


@pytest.mark.parametrize("P,M,v", [(2, 2, 2), (2, 4, 2), (4, 8, 2), (3, 6, 3), (4, 4, 4)])
def test_interleaved_schedule_runs_without_deadlock_and_in_fifo_order(P, M, v):
    """All ranks' step lists executed against first-in-first-out channels: every unit finds its
    input at the head of its channel (the order of sends equals the order of receives) and the
    whole step finishes (no rank waits for a message that is never sent)."""
    V = P * v
    steps = [schedule_interleaved(s, P, M, v) for s in range(P)]
    for s in range(P):
        fs = [(c, i) for k, c, i in steps[s] if k == "F"]
        bs = [(c, i) for k, c, i in steps[s] if k == "B"]
        assert sorted(fs) == sorted(bs) == [(c, i) for c in range(v) for i in range(M)]
    chans = {}                      # (kind, src, dst) -> list of (virtual stage of consumer, mb)
    pc = [0] * P
    done_f, done_b = set(), set()
    progress = True
    while progress:
        progress = False
        for s in range(P):
            while pc[s] < len(steps[s]):
                kind, c, i = steps[s][pc[s]]
                k = c * P + s
                if kind == "F":
                    if k > 0:
                        q = chans.get(("f", (s - 1) % P, s), [])
                        if not q:
                            break
                        assert q.pop(0) == (k, i)
                    if k < V - 1:
                        chans.setdefault(("f", s, (s + 1) % P), []).append((k + 1, i))
                    done_f.add((k, i))
                else:
                    assert (k, i) in done_f
                    if k < V - 1:
                        q = chans.get(("b", (s + 1) % P, s), [])
                        if not q:
                            break
                        assert q.pop(0) == (k, i)
                    if k > 0:
                        chans.setdefault(("b", s, (s - 1) % P), []).append((k - 1, i))
                    done_b.add((k, i))
                pc[s] += 1
                progress = True
    assert all(pc[s] == len(steps[s]) for s in range(P)), "deadlock"
    assert len(done_b) == V * M


def test_launch_order_model_of_nccl_point_to_point():
    """The event model of rendezvous sends and receives: the 1F1B order always finishes, the
    interleaved order only while there are no more micro-batches than stages; the peer-memory
    transport, whose sends never wait, is what the interleaved stage uses on GPUs."""
    for P, M in [(2, 2), (2, 8), (4, 4), (4, 8), (8, 16)]:
        assert not nccl_order_deadlocks(P, M)
    for P, v, M in [(2, 2, 2), (4, 2, 4), (8, 2, 8)]:
        assert not nccl_order_deadlocks(P, M, v)
    for P, v, M in [(2, 2, 4), (2, 4, 8), (4, 2, 8), (3, 3, 9), (8, 2, 16)]:
        assert nccl_order_deadlocks(P, M, v)
    # the order that the model walks is the order of the step loop: every unit computes once,
    # between the receive of its input and the send of its output
    ops = comm_order(1, 4, 8, 2)
    units = [d for kind, d in ops if kind == "compute"]
    assert units == schedule_interleaved(1, 4, 8, 2)
    assert sum(kind == "send" for kind, _ in ops) == sum(kind == "recv" for kind, _ in ops) == 32
    from coeus_b200.foundation.error import ProcessingError
    from coeus_b200.parallel.pp import _check_transport
    with pytest.raises(ProcessingError):
        _check_transport("peer", "cpu")
    with pytest.raises(ProcessingError):
        _check_transport("carrier pigeon", "cpu")


@pytest.mark.parametrize("P,M,v", [(2, 4, 1), (4, 8, 1), (8, 16, 1), (2, 2, 2), (2, 8, 2), (4, 8, 2),
                                   (3, 6, 3), (4, 8, 4), (8, 16, 2)])
def test_ring_depths_hold_under_any_execution_order(P, M, v):
    """The slot counts of the peer-memory transport: with sends that never wait, ranks that run
    in any order (random, and each rank in turn pushed as far ahead as it can go) and several
    steps back to back, a message never lands in a slot whose previous message has not been taken
    yet; and the depths do not grow with the number of micro-batches."""
    import random
    depth = ring_depths(P, M, v)
    assert all(1 <= d <= 2 * P for d in depth.values())
    assert ring_depths(P, 4 * M, v) == depth or M <= P
    steps = 3
    progs = [comm_order(s, P, M, v) * steps for s in range(P)]
    for seed in range(40):
        rng = random.Random(seed)
        favourite = seed % P if seed < 2 * P else None      # this rank runs whenever it can
        pc = [0] * P
        sent, taken = {}, {}
        while any(pc[r] < len(progs[r]) for r in range(P)):
            runnable = []
            for r in range(P):
                if pc[r] == len(progs[r]):
                    continue
                kind, d = progs[r][pc[r]]
                if kind != "recv" or sent.get(d, 0) > taken.get(d, 0):
                    runnable.append(r)
            assert runnable, "the step does not finish with sends that never wait"
            r = favourite if favourite in runnable else rng.choice(runnable)
            kind, d = progs[r][pc[r]]
            if kind == "send":
                n = sent.get(d, 0)
                # slot n % depth held message n - depth: it must have been taken already
                assert n - depth[d[0]] < taken.get(d, 0), (d, n, taken.get(d, 0))
                sent[d] = n + 1
            elif kind == "recv":
                taken[d] = taken.get(d, 0) + 1
            pc[r] += 1
    # the depths are exact: hold back one receipt and run everything that does not depend on it;
    # the sends of its stream that still go out are the ones that may overtake it
    two = [comm_order(s, P, M, v) * 2 for s in range(P)]
    need = {}
    streams = sorted({d for prog in two for kind, d in prog if kind == "recv"})
    for d in streams:
        count = sum(1 for kind, dd in two[d[2]] if kind == "recv" and dd == d)
        for j in range(count // 2):           # receipts of the first step
            pc = [0] * P
            sent, taken = {}, {}
            moved = True
            while moved:
                moved = False
                for r in range(P):
                    while pc[r] < len(two[r]):
                        kind, dd = two[r][pc[r]]
                        if kind == "recv":
                            if dd == d and taken.get(dd, 0) == j:
                                break                         # the receipt that is held back
                            if sent.get(dd, 0) <= taken.get(dd, 0):
                                break
                            taken[dd] = taken.get(dd, 0) + 1
                        elif kind == "send":
                            sent[dd] = sent.get(dd, 0) + 1
                        pc[r] += 1
                        moved = True
            need[d[0]] = max(need.get(d[0], 1), sent.get(d, 0) - j)
    assert need == depth


def _worker_interleaved(rank, world, port, ids, tgt, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from coeus_b200.parallel.pp import InterleavedPipelineStage
    cfg = _cfg()
    cfg.num_layers = 5
    st = InterleavedPipelineStage(cfg, dist.group.WORLD, "cpu", micro_batches=ids.shape[0],
                                  chunks=2, seed=4, dtype=torch.float32, train_cfg=_train_cfg())
    losses = [float(st.train_step(ids, tgt)) for _ in range(2)]
    # checkpoint of an interleaved stage: reload into a differently seeded copy, same next step
    import tempfile
    tmp = os.path.join(tempfile.gettempdir(), f"coeus_ipp_{port}")
    st.save_checkpoint(tmp)
    other = InterleavedPipelineStage(cfg, dist.group.WORLD, "cpu", micro_batches=ids.shape[0],
                                     chunks=2, seed=99, dtype=torch.float32, train_cfg=_train_cfg())
    assert other.load_checkpoint(tmp)["train_step"] == 2
    for a_, b_ in zip(st.models, other.models):
        assert torch.equal(a_.p32, b_.p32)
    # on GPUs the NCCL transport is refused where its launch order can stop (no device is touched
    # before that check), and a CPU rank cannot ask for the peer-memory transport
    from coeus_b200.foundation.error import ProcessingError
    assert ids.shape[0] > world
    with pytest.raises(ProcessingError):
        InterleavedPipelineStage(cfg, dist.group.WORLD, "cuda", micro_batches=ids.shape[0],
                                 chunks=2, transport="nccl")
    with pytest.raises(ProcessingError):
        InterleavedPipelineStage(cfg, dist.group.WORLD, "cpu", micro_batches=ids.shape[0],
                                 chunks=2, transport="peer")
    params = {}
    for m in st.models:
        params.update({k: v.numpy().copy() for k, v in m.master.items()})
    out.put((rank, losses, params))
    dist.barrier()
    dist.destroy_process_group()


def test_interleaved_pipeline_training_matches_single_rank():
    from mp_util import run_ranks
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.optim.adamw import AdamW
    torch.manual_seed(0)
    M, b, S, world = 4, 2, 16, 2
    ids = torch.randint(0, 96, (M, b, S))
    tgt = torch.randint(0, 96, (M, b, S))
    cfg = _cfg()
    cfg.num_layers = 5
    full = DecoderLM(cfg, "cpu", seed=4, dtype=torch.float32)
    opt = AdamW(_train_cfg().adamw(), 0, full.n_flat, full.layout.decay_end, "cpu")
    ref_losses = []
    for _ in range(2):
        full.zero_grad()
        tot = 0.0
        for i in range(M):
            tot += float(full.forward_loss(ids[i], tgt[i], grad_scale=1.0 / (b * S * M))) / M
            full.backward()
        opt.step(full.p32, full.g32, full.p16, 1.0)
        ref_losses.append(tot)
    res = {r[0]: r for r in run_ranks(_worker_interleaved, world, (ids, tgt), results=world)}
    for step in range(2):
        assert abs(res[world - 1][1][step] - ref_losses[step]) < 1e-5
    seen = set()
    for rank in range(world):
        for name, got in res[rank][2].items():
            assert (torch.from_numpy(got) - full.master[name]).abs().max() < 1e-5, name
            seen.add(name)
    assert seen == set(full.master)


def _worker_ckpt(rank, world, port, ids, tgt, tmp, mode, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from coeus_b200.parallel.pp import PipelineStage
    st = PipelineStage(_cfg(), dist.group.WORLD, "cpu", micro_batches=ids.shape[0],
                       seed=4 if mode == "save" else 11, dtype=torch.float32, train_cfg=_train_cfg())
    if mode == "save":
        for _ in range(2):
            st.train_step(ids, tgt)
        st.save_checkpoint(tmp)
        loss = 0.0
    else:
        man = st.load_checkpoint(tmp)
        assert man["train_step"] == 2 and man["stages"] == 2
        loss = float(st.train_step(ids, tgt))
    out.put((rank, loss))
    dist.barrier()
    dist.destroy_process_group()


def test_pipeline_checkpoint_resumes_on_another_number_of_stages(tmp_path):
    """Saved by two stages, resumed by three stages and by a single process: the third step is
    the third step of the single-rank run."""
    from mp_util import run_ranks
    from coeus_b200.checkpoint.named import load_named, model_state
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.optim.adamw import AdamW
    torch.manual_seed(0)
    M, b, S = 4, 2, 16
    ids = torch.randint(0, 96, (M, b, S))
    tgt = torch.randint(0, 96, (M, b, S))
    full = DecoderLM(_cfg(), "cpu", seed=4, dtype=torch.float32)
    opt = AdamW(_train_cfg().adamw(), 0, full.n_flat, full.layout.decay_end, "cpu")

    def ref_step(model, o):
        model.zero_grad()
        tot = 0.0
        for i in range(M):
            tot += float(model.forward_loss(ids[i], tgt[i], grad_scale=1.0 / (b * S * M))) / M
            model.backward()
        o.step(model.p32, model.g32, model.p16, 1.0)
        return tot
    for _ in range(2):
        ref_step(full, opt)
    run_ranks(_worker_ckpt, 2, (ids, tgt, str(tmp_path), "save"), results=2)
    # single process
    one = DecoderLM(_cfg(), "cpu", seed=11, dtype=torch.float32)
    o1 = AdamW(_train_cfg().adamw(), 0, one.n_flat, one.layout.decay_end, "cpu")
    man = load_named(str(tmp_path), model_state(one, o1))
    one.sync_working_copy()
    o1.step_count = int(man["opt_step"])
    assert (one.p32 - full.p32).abs().max() < 1e-5 and (o1.v - opt.v).abs().max() < 1e-6
    want = ref_step(full, opt)
    assert abs(ref_step(one, o1) - want) < 1e-5
    # three stages
    res = {r[0]: r[1] for r in run_ranks(_worker_ckpt, 3, (ids, tgt, str(tmp_path), "load"),
                                         results=3)}
    assert abs(res[2] - want) < 1e-5


def test_peer_ring_addresses_and_sequence_numbers(monkeypatch):
    """The two ends of a peer-memory stream agree on where message n lives and what its flag
    says: checked against a recording stand-in for the kernel library and the symmetric buffer
    (no GPU): the sender's destination is the receiver's slot n mod depth, the flag raised is the
    one waited for, its value is n + 1, and the regions of the four kinds of stream are disjoint."""
    import ctypes
    import coeus_b200.parallel.pp as pp
    import coeus_b200.parallel.symm as symm
    from coeus_b200.ops import _lib

    bases = [0x10000000, 0x20000000]
    calls = []

    class FakeBuffer:
        def __init__(self, nbytes, group, device):
            self.nbytes, self.rank = nbytes, group
            self.ptrs = list(bases)
            self.local_ptr = bases[group]

        def view(self, dtype, byte_offset=0, numel=None):
            calls.append(("view", self.rank, byte_offset, numel))
            return torch.zeros(numel, dtype=dtype)

        def close(self):
            pass

    def val(x):
        return x.value if hasattr(x, "value") else int(x)

    class FakeLib:
        def cb_peer_copy(self, src, dst, nbytes, blocks, stream):
            calls.append(("copy", val(dst), val(nbytes)))
            return 0

        def cb_signal_peers(self, flags, slot, n, my_rank, value, stream):
            assert (slot, n, my_rank) == (0, 1, 0)
            calls.append(("signal", int(flags[0]), val(value)))
            return 0

        def cb_wait_flags(self, flag, slot, n, value, limit, status, stream):
            assert (slot, n) == (0, 1)
            calls.append(("wait", val(flag), val(value)))
            return 0

    monkeypatch.setattr(symm, "SymmetricBuffer", FakeBuffer)
    monkeypatch.setattr(_lib, "lib", lambda: FakeLib())
    monkeypatch.setattr(_lib, "stream_ptr", lambda: ctypes.c_void_p(0))
    monkeypatch.setattr(_lib, "status_buffer", lambda device: None)
    depths = {"f": 3, "b": 2, "fw": 2, "bw": 1}
    shape, dtype = (6, 40), torch.bfloat16            # 480 bytes: a slot is padded to 512
    send = pp.PeerRing(0, "cpu", shape, dtype, depths, copy_out=True)     # "group" = rank here
    recv = pp.PeerRing(1, "cpu", shape, dtype, depths, copy_out=True)
    assert send.slot_bytes == 512 and send.data_off == recv.data_off
    regions = sorted((send.data_off[k], send.data_off[k] + depths[k] * 512) for k in depths)
    assert all(a[1] <= b[0] for a, b in zip(regions, regions[1:]))
    assert min(send.flag_off.values()) >= regions[-1][1]
    t = torch.zeros(shape, dtype=dtype)
    for n in range(7):
        calls.clear()
        send.push("f", 1, t)
        got = recv.take("f")
        assert got.shape == shape
        copy, signal, wait, view = calls
        slot = n % 3
        assert copy == ("copy", bases[1] + send.data_off["f"] + slot * 512, 480)
        assert signal == ("signal", bases[1] + send.flag_off["f"] + slot * 8, n + 1)
        assert wait == ("wait", signal[1], n + 1)
        assert view == ("view", 1, recv.data_off["f"] + slot * 512, 240)
    # another kind of stream counts on its own and lives elsewhere
    calls.clear()
    send.push("bw", 1, t)
    assert calls[0][1] == bases[1] + send.data_off["bw"] and calls[1][2] == 1
