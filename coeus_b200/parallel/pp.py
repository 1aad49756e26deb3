"""Pipeline parallelism: the decoder's blocks are split into contiguous stages, one per rank, and
micro-batches flow through them in the one-forward-one-backward (1F1B) order.

Stage ``s`` of ``P`` runs ``min(P - 1 - s, M)`` warm-up forwards, then alternates one forward and
one backward, then drains the remaining backwards; at most ``P - s`` micro-batches are alive on a
stage at a time, which bounds the activation stash.  Activations and their gradients travel with
point-to-point sends (NCCL on GPUs, Gloo on CPU ranks).  The forward and the backward direction
use separate process groups, so a receive that was posted early never blocks a send of the other
direction; sends are not waited for until their buffer is reused and, on CPU ranks, receives for
the next micro-batch are posted before the current one is computed (on GPUs a receive is posted
when it is needed, see ``_Channel``), which is what overlaps the transfers with the math.  The reference is a single process and has no pipeline (no send/recv anywhere in its
sources); this is one of the parallelism strategies the larger training configurations need.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..foundation.error import ProcessingError
from ..models.config import DecoderConfig
from ..models.decoder import DecoderLM
from ..ops import elementwise as E


def split_layers(num_layers: int, stages: int) -> List[Tuple[int, int]]:
    """Contiguous ``(lo, hi)`` block ranges, the remainder going to the earliest stages."""
    if stages < 1 or stages > num_layers:
        raise ProcessingError.invalid_input(
            f"cannot split {num_layers} layers into {stages} pipeline stages")
    base, rem = divmod(num_layers, stages)
    out, lo = [], 0
    for s in range(stages):
        hi = lo + base + (1 if s < rem else 0)
        out.append((lo, hi))
        lo = hi
    return out


def schedule_1f1b(stage: int, stages: int, micro_batches: int) -> List[Tuple[str, int]]:
    """The order of ``("F", i)`` / ``("B", i)`` steps of one stage."""
    warm = min(stages - 1 - stage, micro_batches)
    steps: List[Tuple[str, int]] = [("F", i) for i in range(warm)]
    f, b = warm, 0
    while f < micro_batches:
        steps.append(("F", f))
        steps.append(("B", b))
        f += 1
        b += 1
    while b < micro_batches:
        steps.append(("B", b))
        b += 1
    return steps


def schedule_interleaved(stage: int, stages: int, micro_batches: int, chunks: int
                         ) -> List[Tuple[str, int, int]]:
    """Interleaved 1F1B: every rank holds ``chunks`` model chunks (chunk ``c`` of rank ``s`` is
    virtual stage ``c * stages + s``), which shortens the pipeline bubble by the factor ``chunks``.
    Returns ``("F" | "B", chunk, micro_batch)`` steps.  Forward units advance in groups of
    ``stages`` micro-batches through chunk 0, 1, ...; backward units through the chunks in
    reverse; ``micro_batches`` must be a multiple of ``stages``."""
    P, M, v = stages, micro_batches, chunks
    if M % P:
        raise ProcessingError.invalid_input(
            "the interleaved schedule needs micro_batches to be a multiple of the stage count")
    total = M * v

    def unit(n: int, backward: bool) -> Tuple[int, int]:
        c = (n // P) % v
        return (v - 1 - c if backward else c), (n // (P * v)) * P + n % P

    warm = min((P - stage - 1) * 2 + (v - 1) * P, total)
    steps: List[Tuple[str, int, int]] = [("F",) + unit(n, False) for n in range(warm)]
    f, b = warm, 0
    while f < total:
        steps.append(("F",) + unit(f, False))
        steps.append(("B",) + unit(b, True))
        f += 1
        b += 1
    while b < total:
        steps.append(("B",) + unit(b, True))
        b += 1
    return steps


class _Channel:
    """One direction between two neighbouring stages: posts receives ahead and keeps sends alive."""

    def __init__(self, group, peer_global: int, shape, dtype, device, count: int, recv: bool) -> None:
        # Receives are posted ahead only on CPU ranks.  On a GPU an early NCCL receive is a kernel
        # that spins on its SMs until the peer sends; the persistent GEMM kernels (one CTA per SM,
        # static tile assignment) cannot place their CTAs there, and two neighbouring stages that
        # both wait like this for each other's next tensor would never finish the GEMMs that
        # produce them.  So on CUDA a receive is posted when its tensor is needed, sends stay
        # asynchronous.
        self.prefetch = torch.device(device).type != "cuda"
        self.group, self.peer, self.count = group, peer_global, count
        self.shape, self.dtype, self.device = shape, dtype, device
        self.posted = 0
        self.pending: List[Tuple[object, torch.Tensor]] = []
        self.recv = recv

    def post_recv(self, force: bool = False) -> None:
        if self.posted >= self.count or not (self.prefetch or force):
            return
        buf = torch.empty(self.shape, dtype=self.dtype, device=self.device)
        self.pending.append((dist.irecv(buf, src=self.peer, group=self.group), buf))
        self.posted += 1

    def take(self) -> torch.Tensor:
        if not self.pending:
            self.post_recv(force=True)
        req, buf = self.pending.pop(0)
        req.wait()
        self.post_recv()          # the next one travels while this one is computed on
        return buf

    def send(self, t: torch.Tensor) -> None:
        t = t.contiguous()
        self.pending.append((dist.isend(t, dst=self.peer, group=self.group), t))
        while len(self.pending) > 2:     # bound the number of buffers kept alive
            req, _ = self.pending.pop(0)
            req.wait()

    def drain(self) -> None:
        for req, _ in self.pending:
            req.wait()
        self.pending.clear()


class PipelineStage:
    """One rank's share of a pipelined decoder plus the 1F1B step loop."""

    def __init__(self, cfg: DecoderConfig, group, device, micro_batches: int, seed: int = 0,
                 dtype: torch.dtype = torch.bfloat16, train_cfg=None, schedule=None) -> None:
        from ..optim.adamw import AdamW
        from ..train.trainer import TrainConfig
        self.schedule = schedule          # object with at(step) -> learning rate
        self.group = group
        self.stage = dist.get_rank(group) if group is not None else 0
        self.stages = dist.get_world_size(group) if group is not None else 1
        self.M = micro_batches
        self.device = torch.device(device)
        lo, hi = split_layers(cfg.num_layers, self.stages)[self.stage]
        self.first, self.last = self.stage == 0, self.stage == self.stages - 1
        self.model = DecoderLM(cfg, self.device, seed=seed, dtype=dtype, layers=(lo, hi),
                               embed=self.first, head=self.last)
        self.cfg = cfg
        self.train_cfg = train_cfg or TrainConfig()
        self.opt = AdamW(self.train_cfg.adamw(), 0, self.model.n_flat, self.model.layout.decay_end,
                         self.device)
        if self.stages > 1:
            ranks = dist.get_process_group_ranks(group)
            # two groups: traffic of one direction never queues behind the other
            self.fwd_group = dist.new_group(ranks)
            self.bwd_group = dist.new_group(ranks)
            self._ranks = ranks
            # global gradient norm: every stage holds its own tensors
            self.opt.norm_hook = lambda g32, sumsq: dist.all_reduce(sumsq, group=self.group)
        self.step_index = 0

    def load_from_full(self, full: DecoderLM) -> None:
        """Copy this stage's tensors out of a model that holds every layer."""
        for name, t in self.model.master.items():
            t.copy_(full.master[name])
        self.model.sync_working_copy()

    def save_checkpoint(self, directory: str) -> None:
        """Name-keyed training checkpoint (weights and Adam moments of this stage's tensors);
        loads into any number of stages."""
        from ..checkpoint.named import model_state, save_named
        barrier = (lambda: dist.barrier(group=self.group)) if self.stages > 1 else None
        save_named(directory, self.stage, model_state(self.model, self.opt),
                   {"stages": self.stages, "opt_step": self.opt.step_count,
                    "train_step": self.step_index, "config": self.cfg.to_dict()}, barrier)

    def load_checkpoint(self, directory: str) -> dict:
        from ..checkpoint.named import load_named, model_state
        man = load_named(directory, model_state(self.model, self.opt))
        self.model.sync_working_copy()
        self.opt.step_count = int(man["opt_step"])
        self.step_index = int(man["train_step"])
        return man

    def train_step(self, ids: Optional[torch.Tensor], targets: Optional[torch.Tensor]) -> torch.Tensor:
        """One optimizer step over ``M`` micro-batches.  ``ids [M, b, S]`` is needed on the first
        stage, ``targets [M, b, S]`` on the last; both may be given everywhere.  Returns the mean
        loss on the last stage (zeros elsewhere)."""
        m, M = self.model, self.M
        ref = ids if ids is not None else targets
        b, S = ref.shape[1], ref.shape[2]
        T, H = b * S, self.cfg.hidden_dim
        act_dtype = m.p16.dtype
        chans: Dict[str, _Channel] = {}
        if self.stages > 1:
            if not self.first:
                chans["rf"] = _Channel(self.fwd_group, self._ranks[self.stage - 1], (T, H),
                                       act_dtype, self.device, M, True)
                chans["sb"] = _Channel(self.bwd_group, self._ranks[self.stage - 1], (T, H),
                                       act_dtype, self.device, M, False)
            if not self.last:
                chans["sf"] = _Channel(self.fwd_group, self._ranks[self.stage + 1], (T, H),
                                       act_dtype, self.device, M, False)
                chans["rb"] = _Channel(self.bwd_group, self._ranks[self.stage + 1], (T, H),
                                       act_dtype, self.device, M, True)
        m.zero_grad()
        saves: Dict[int, dict] = {}
        loss_sum = torch.zeros(1, dtype=torch.float32, device=self.device)
        if "rf" in chans:
            chans["rf"].post_recv()
        for kind, i in schedule_1f1b(self.stage, self.stages, M):
            m._ws_tag = f"mb{i % (self.stages - self.stage)}:"   # slots of micro-batches in flight
            if kind == "F":
                save: dict = {"B": b, "S": S}
                if self.first:
                    flat = ids[i].reshape(-1)
                    save["ids"] = flat
                    x = m.embed(ids[i], b, S)
                else:
                    x = chans["rf"].take()
                x = m.forward_blocks(x, b, S, save)
                if self.last:
                    xf = m.forward_final_norm(x, save)
                    loss = m.loss_from_hidden(xf, targets[i], save, grad_scale=1.0 / (T * M))
                    loss_sum += loss / M
                else:
                    chans["sf"].send(x)
                saves[i] = save
                if "rb" in chans and not chans["rb"].pending:
                    chans["rb"].post_recv()
            else:
                save = saves.pop(i)
                dx = m.backward_head(save) if self.last else chans["rb"].take()
                dx = m.backward_blocks(dx, save)
                if self.first:
                    E.embed_bwd(save["ids"], dx, m.g["token_embed"])
                    m.backward_positions(dx, save)
                else:
                    chans["sb"].send(dx)
        for c in chans.values():
            c.drain()
        m._ws_tag = ""
        if self.schedule is not None:
            self.opt.set_learning_rate(self.schedule.at(self.step_index))
        self.opt.step(m.p32, m.g32, m.p16, 1.0)
        self.step_index += 1
        return loss_sum


class InterleavedPipelineStage:
    """One rank of a pipeline whose ranks each hold ``chunks`` non-adjacent groups of blocks
    (virtual stages), run in the interleaved 1F1B order of :func:`schedule_interleaved`.

    Activations travel round the ring of ranks: from rank ``s`` to ``s + 1`` inside one chunk and
    from the last rank back to the first between chunks; gradients go the other way.  The four
    kinds of transfer (forward / backward, inside a chunk / between chunks) use four process
    groups, so each is a first-in-first-out stream whose order is the same on its two ends (both
    follow the order of the schedule's units) and a transfer of one kind never queues behind one
    of another kind.  On GPUs receives are posted when needed (see ``_Channel``)."""

    def __init__(self, cfg: DecoderConfig, group, device, micro_batches: int, chunks: int = 2,
                 seed: int = 0, dtype: torch.dtype = torch.bfloat16, train_cfg=None,
                 schedule=None) -> None:
        from ..optim.adamw import AdamW
        from ..train.trainer import TrainConfig
        self.schedule = schedule
        self.group = group
        self.stage = dist.get_rank(group)
        self.stages = dist.get_world_size(group)
        if self.stages < 2 or chunks < 2:
            raise ProcessingError.invalid_input(
                "the interleaved pipeline needs at least two ranks and two chunks per rank")
        self.M, self.v, self.cfg = micro_batches, chunks, cfg
        self.device = torch.device(device)
        P, V = self.stages, self.stages * chunks
        spans = split_layers(cfg.num_layers, V)
        self.models: List[DecoderLM] = []
        self.opts = []
        self.train_cfg = train_cfg or TrainConfig()
        for c in range(chunks):
            k = c * P + self.stage
            m = DecoderLM(cfg, self.device, seed=seed, dtype=dtype, layers=spans[k],
                          embed=(k == 0), head=(k == V - 1))
            self.models.append(m)
            self.opts.append(AdamW(self.train_cfg.adamw(), 0, m.n_flat, m.layout.decay_end,
                                   self.device))
        ranks = dist.get_process_group_ranks(group)
        self._ranks = ranks
        self._groups = {k: dist.new_group(ranks) for k in ("f", "fw", "b", "bw")}
        self.steps = schedule_interleaved(self.stage, P, micro_batches, chunks)
        # workspace slots: micro-batches of one chunk that are alive together never share one
        self._slot: Dict[Tuple[int, int], int] = {}
        free = [list() for _ in range(chunks)]
        used = [0] * chunks
        for kind, c, i in self.steps:
            if kind == "F":
                if free[c]:
                    self._slot[(c, i)] = free[c].pop()
                else:
                    self._slot[(c, i)] = used[c]
                    used[c] += 1
            else:
                free[c].append(self._slot[(c, i)])
        self.step_index = 0

    def load_from_full(self, full: DecoderLM) -> None:
        for m in self.models:
            for name, t in m.master.items():
                t.copy_(full.master[name])
            m.sync_working_copy()

    def _virtual(self, c: int) -> int:
        return c * self.stages + self.stage

    def _state(self) -> dict:
        from ..checkpoint.named import model_state
        st: dict = {}
        for m, opt in zip(self.models, self.opts):
            st.update(model_state(m, opt))
        return st

    def save_checkpoint(self, directory: str) -> None:
        """Name-keyed checkpoint of all chunks of this rank; loads into any pipeline shape."""
        from ..checkpoint.named import save_named
        save_named(directory, self.stage, self._state(),
                   {"stages": self.stages, "chunks": self.v, "opt_step": self.opts[0].step_count,
                    "train_step": self.step_index, "config": self.cfg.to_dict()},
                   lambda: dist.barrier(group=self.group))

    def load_checkpoint(self, directory: str) -> dict:
        from ..checkpoint.named import load_named
        man = load_named(directory, self._state())
        for m, opt in zip(self.models, self.opts):
            m.sync_working_copy()
            opt.step_count = int(man["opt_step"])
        self.step_index = int(man["train_step"])
        return man

    def train_step(self, ids: Optional[torch.Tensor], targets: Optional[torch.Tensor]) -> torch.Tensor:
        """One optimizer step over ``M`` micro-batches; ``ids [M, b, S]`` is read on the first
        rank, ``targets`` on the last.  Returns the mean loss on the last rank."""
        P, v, M, s = self.stages, self.v, self.M, self.stage
        V = P * v
        ref = ids if ids is not None else targets
        b, S = ref.shape[1], ref.shape[2]
        T, H = b * S, self.cfg.hidden_dim
        dt = self.models[0].p16.dtype
        nxt, prv = self._ranks[(s + 1) % P], self._ranks[(s - 1) % P]
        n_wrap = M * (v - 1)

        def chan(key, peer, count, recv):
            return _Channel(self._groups[key], peer, (T, H), dt, self.device, count, recv)

        ch: Dict[str, _Channel] = {}
        if s > 0:                       # inside a chunk: s-1 -> s forward, s -> s-1 backward
            ch["rf"] = chan("f", prv, M * v, True)
            ch["sb"] = chan("b", prv, M * v, False)
        if s < P - 1:
            ch["sf"] = chan("f", nxt, M * v, False)
            ch["rb"] = chan("b", nxt, M * v, True)
        if s == P - 1:                  # between chunks: last -> first forward, first -> last backward
            ch["sfw"] = chan("fw", nxt, n_wrap, False)
            ch["rbw"] = chan("bw", nxt, n_wrap, True)
        if s == 0:
            ch["rfw"] = chan("fw", prv, n_wrap, True)
            ch["sbw"] = chan("bw", prv, n_wrap, False)
        for m in self.models:
            m.zero_grad()
        saves: Dict[Tuple[int, int], dict] = {}
        loss_sum = torch.zeros(1, dtype=torch.float32, device=self.device)
        for kind, c, i in self.steps:
            m, k = self.models[c], self._virtual(c)
            m._ws_tag = f"mb{self._slot[(c, i)]}:"
            if kind == "F":
                save: dict = {"B": b, "S": S}
                if k == 0:
                    save["ids"] = ids[i].reshape(-1)
                    x = m.embed(ids[i], b, S)
                else:
                    x = ch["rf" if s > 0 else "rfw"].take()
                x = m.forward_blocks(x, b, S, save)
                if k == V - 1:
                    xf = m.forward_final_norm(x, save)
                    loss = m.loss_from_hidden(xf, targets[i], save, grad_scale=1.0 / (T * M))
                    loss_sum += loss / M
                else:
                    ch["sf" if s < P - 1 else "sfw"].send(x)
                saves[(c, i)] = save
            else:
                save = saves.pop((c, i))
                if k == V - 1:
                    dx = m.backward_head(save)
                else:
                    dx = ch["rb" if s < P - 1 else "rbw"].take()
                dx = m.backward_blocks(dx, save)
                if k == 0:
                    E.embed_bwd(save["ids"], dx, m.g["token_embed"])
                    m.backward_positions(dx, save)
                else:
                    ch["sb" if s > 0 else "sbw"].send(dx)
        for c_ in ch.values():
            c_.drain()
        if self.train_cfg.grad_clip is not None:
            # one norm over all chunks of all ranks, handed to every chunk's optimizer
            total = torch.zeros(1, dtype=torch.float32, device=self.device)
            for m in self.models:
                E.sumsq_into(m.g32, total)
            dist.all_reduce(total, group=self.group)
            for opt in self.opts:
                opt.norm_hook = lambda g32, sumsq, t=total: sumsq.copy_(t)
        for m, opt in zip(self.models, self.opts):
            m._ws_tag = ""
            if self.schedule is not None:
                opt.set_learning_rate(self.schedule.at(self.step_index))
            opt.step(m.p32, m.g32, m.p16, 1.0)
        self.step_index += 1
        return loss_sum
