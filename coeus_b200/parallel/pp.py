"""Pipeline parallelism: the decoder's blocks are split into contiguous stages, one per rank, and
micro-batches flow through them in the one-forward-one-backward (1F1B) order.

Stage ``s`` of ``P`` runs ``min(P - 1 - s, M)`` warm-up forwards, then alternates one forward and
one backward, then drains the remaining backwards; at most ``P - s`` micro-batches are alive on a
stage at a time, which bounds the activation stash.  Activations and their gradients travel with
point-to-point sends (NCCL on GPUs, Gloo on CPU ranks).  The forward and the backward direction
use separate process groups, so a receive that was posted early never blocks a send of the other
direction; sends are not waited for until their buffer is reused and, on CPU ranks, receives for
the next micro-batch are posted before the current one is computed (on GPUs a receive is posted
when it is needed, see ``_Channel``), which is what overlaps the transfers with the math.  The
reference is a single process and has no pipeline (no send/recv anywhere in its sources); this
is one of the parallelism strategies the larger training configurations need.

On GPUs there is a second transport, ``transport="peer"``: the sender pushes the tensor into a
slot of the receiver's memory over NVLink (a copy kernel on the compute stream followed by a
release store of the slot's 64-bit flag, the message's sequence number), the receiver's stream
waits for the flag with a bounded spin of one warp and copies the tensor out of the slot (or,
with a slot per message of a step, computes straight out of it).  The number of slots comes
from the step's own order of sends and receipts (:func:`ring_depths`).  Nothing is a
rendezvous: a send never waits for the receiver to have posted anything, so any schedule that
finishes with asynchronous sends finishes.  NCCL point-to-point is a rendezvous of two kernels, and a spinning NCCL kernel
can hold back the compute kernels queued behind it; :func:`nccl_order_deadlocks` is an event
model of that, under which the interleaved schedule stops for ``micro_batches > stages`` (two
ranks each spin in a send whose receive the other rank posts only after compute that the spin
holds back).  The interleaved stage therefore uses the peer transport on GPUs.
"""
from __future__ import annotations

import functools
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


def comm_order(stage: int, stages: int, micro_batches: int, chunks: int = 1
               ) -> List[Tuple[str, tuple]]:
    """The order in which one rank's ``train_step`` issues receives, compute units and sends:
    ``("recv" | "send", (kind, src, dst))`` and ``("compute", unit)``.  ``kind`` names the stream of
    messages (``f`` / ``b`` inside a chunk, ``fw`` / ``bw`` between chunks)."""
    P, V, s = stages, stages * chunks, stage
    if chunks == 1:
        units = [(kind, 0, i) for kind, i in schedule_1f1b(s, P, micro_batches)]
    else:
        units = schedule_interleaved(s, P, micro_batches, chunks)
    ops: List[Tuple[str, tuple]] = []
    for kind, c, i in units:
        k = c * P + s
        if kind == "F":
            if k != 0:
                ops.append(("recv", ("f" if s > 0 else "fw", (s - 1) % P, s)))
            ops.append(("compute", (kind, c, i)))
            if k != V - 1:
                ops.append(("send", ("f" if s < P - 1 else "fw", s, (s + 1) % P)))
        else:
            if k != V - 1:
                ops.append(("recv", ("b" if s < P - 1 else "bw", (s + 1) % P, s)))
            ops.append(("compute", (kind, c, i)))
            if k != 0:
                ops.append(("send", ("b" if s > 0 else "bw", s, (s - 1) % P)))
    return ops


def nccl_order_deadlocks(stages: int, micro_batches: int, chunks: int = 1) -> bool:
    """Event model of :func:`comm_order` run with NCCL point-to-point kernels on GPUs.

    A send or receive kernel starts once the compute issued before it is done and the previous
    message between the same two ranks in the same group is through; it finishes once its
    counterpart on the other rank has started (a rendezvous).  A compute unit starts when the
    compute before it is done, its input has arrived and no communication kernel that this rank
    has started is still spinning (the pessimistic part: a spinning kernel is assumed to hold back
    the kernels queued behind it).  Returns True when some rank cannot finish its list."""
    ranks = [comm_order(s, stages, micro_batches, chunks) for s in range(stages)]
    started = [[False] * len(r) for r in ranks]
    finished = [[False] * len(r) for r in ranks]
    sends: Dict[tuple, list] = {}
    recvs: Dict[tuple, list] = {}
    for r, ops in enumerate(ranks):
        for idx, (kind, d) in enumerate(ops):
            if kind == "send":
                sends.setdefault(d, []).append((r, idx))
            elif kind == "recv":
                recvs.setdefault(d, []).append((r, idx))
    peer = {}
    for d, lst in sends.items():
        for a, b in zip(lst, recvs[d]):
            peer[a], peer[b] = b, a
    progress = True
    while progress:
        progress = False
        for r, ops in enumerate(ranks):
            for idx, (kind, d) in enumerate(ops):
                if finished[r][idx]:
                    continue
                if not started[r][idx]:
                    ok = all(finished[r][j] for j in range(idx) if ops[j][0] == "compute")
                    if kind == "compute":
                        ok = ok and all(finished[r][j] for j in range(idx)
                                        if ops[j][0] == "recv" or started[r][j])
                    else:
                        key = (d[0], frozenset(d[1:]))
                        ok = ok and all(finished[r][j] for j in range(idx)
                                        if ops[j][0] != "compute"
                                        and (ops[j][1][0], frozenset(ops[j][1][1:])) == key)
                    if ok:
                        started[r][idx] = progress = True
                        if kind == "compute":
                            finished[r][idx] = True
                if started[r][idx] and not finished[r][idx] and started[peer[(r, idx)][0]][peer[(r, idx)][1]]:
                    finished[r][idx] = progress = True
    return not all(all(f) for f in finished)


def ring_depths(stages: int, micro_batches: int, chunks: int = 1) -> Dict[str, int]:
    """See :func:`_ring_depths` (this wrapper keeps the results of earlier calls)."""
    return dict(_ring_depths_cached(stages, micro_batches, chunks))


@functools.lru_cache(maxsize=None)
def _ring_depths_cached(stages: int, micro_batches: int, chunks: int) -> tuple:
    return tuple(sorted(_ring_depths(stages, micro_batches, chunks).items()))


def _ring_depths(stages: int, micro_batches: int, chunks: int = 1) -> Dict[str, int]:
    """How many receive slots a stream of messages needs when the receiver copies a message out
    of its slot as it takes it and nothing is acknowledged.

    Message ``k`` of a stream may overwrite message ``j`` (``k > j``) only if its send is ordered
    after the receipt of ``j`` by the step's own dependencies: program order on each rank plus
    "a message is received after it is sent".  For every receipt the earliest point of every
    rank's program that is ordered after it is propagated to a fixed point; the first later send
    of the stream at or past the sender's point gives the distance that is safe for ``j``, and the
    depth of a kind of stream (``f`` / ``b`` inside a chunk, ``fw`` / ``bw`` between chunks) is
    the largest distance over its messages and ranks.  A receipt that no later send of the step
    follows is followed by the next step's first message (all of a step's receipts precede the
    next step's sends: its forward traffic starts at the first rank, which finishes a step last,
    and its backward traffic follows that forward traffic), i.e. by the message ``count - j``
    places on."""
    ranks = [comm_order(s, stages, micro_batches, chunks) for s in range(stages)]
    sends: Dict[tuple, list] = {}
    recvs: Dict[tuple, list] = {}
    for r, ops in enumerate(ranks):
        for idx, (kind, d) in enumerate(ops):
            if kind == "send":
                sends.setdefault(d, []).append((r, idx))
            elif kind == "recv":
                recvs.setdefault(d, []).append((r, idx))
    # for every send event, the receive it lands in
    lands: List[Dict[int, Tuple[int, int]]] = [dict() for _ in ranks]
    for d, lst in sends.items():
        for (r, idx), dest in zip(lst, recvs[d]):
            lands[r][idx] = dest
    send_idx = [sorted(m) for m in lands]
    depth: Dict[str, int] = {}
    for d, rlist in recvs.items():
        slist = sends[d]
        sender = slist[0][0]
        need = 1
        for j, (r0, i0) in enumerate(rlist):
            earliest = [len(ops) for ops in ranks]       # first op of each rank ordered after
            earliest[r0] = i0 + 1
            done_from = [len(ops) for ops in ranks]      # sends at or past this index are relaxed
            changed = True
            while changed:
                changed = False
                for r in range(stages):
                    if earliest[r] < done_from[r]:
                        for idx in send_idx[r]:
                            if earliest[r] <= idx < done_from[r]:
                                rr, ii = lands[r][idx]
                                if ii + 1 < earliest[rr]:
                                    earliest[rr] = ii + 1
                        done_from[r] = earliest[r]
                        changed = True
            k = next((k for k in range(j + 1, len(slist)) if slist[k][1] >= earliest[sender]),
                     len(slist))
            need = max(need, k - j)
        depth[d[0]] = max(depth.get(d[0], 1), need)
    return depth


class PeerRing:
    """Receive slots of one rank for the pipeline's message streams, in a symmetric NVLink-mapped
    buffer: ``depths[kind]`` slots of one activation tensor each plus one 64-bit flag per slot.

    Both ends of a stream count its messages (over all steps): message ``n`` goes to slot
    ``n % depth`` and raises that slot's flag to ``n + 1``; the receiver's stream waits for the
    flag to reach ``n + 1``.  With ``copy_out`` the receiver copies the tensor out of the slot as
    it takes it, and the depth only has to cover the messages whose send is not ordered after
    that receipt (:func:`ring_depths`); without it the tensor is used in place for the rest of
    the step, and the depth is the number of messages of a step.  Either way no acknowledgement
    travels back: the pipeline's own data dependencies order every overwrite after the last read
    of what it overwrites."""

    KINDS = ("f", "b", "fw", "bw")

    def __init__(self, group, device, shape, dtype, depths: Dict[str, int],
                 limit_ms: float = 30000.0, copy_out: bool = False) -> None:
        from .symm import SymmetricBuffer
        self.shape, self.dtype = tuple(shape), dtype
        self.numel = 1
        for n in self.shape:
            self.numel *= n
        item = torch.empty((), dtype=dtype).element_size()
        self.slot_bytes = (self.numel * item + 255) // 256 * 256
        self.depths = {k: int(depths.get(k, 0)) for k in self.KINDS}
        self.copy_out = copy_out
        self.data_off, self.flag_off = {}, {}
        off = 0
        for k in self.KINDS:
            self.data_off[k] = off
            off += self.depths[k] * self.slot_bytes
        for k in self.KINDS:
            self.flag_off[k] = off
            off += (self.depths[k] * 8 + 255) // 256 * 256
        self.buf = SymmetricBuffer(max(off, 256), group, torch.device(device))
        self.device = torch.device(device)
        self.limit_ns = int(limit_ms * 1e6)
        self.copy_bytes = self.numel * item
        self.sent = {k: 0 for k in self.KINDS}       # messages pushed / taken so far, per stream
        self.taken = {k: 0 for k in self.KINDS}

    def push(self, kind: str, peer: int, t: torch.Tensor) -> None:
        """Copy ``t`` into the next slot of stream ``kind`` on group rank ``peer``, raise its flag."""
        import ctypes
        from ..ops import _lib
        t = t.contiguous()
        lib = _lib.lib()
        n = self.sent[kind]
        slot = n % self.depths[kind]
        self.sent[kind] = n + 1
        dst = self.buf.ptrs[peer] + self.data_off[kind] + slot * self.slot_bytes
        nbytes = (self.copy_bytes + 15) // 16 * 16
        rc = lib.cb_peer_copy(_lib.ptr(t), ctypes.c_void_p(dst), ctypes.c_size_t(nbytes), 0,
                              _lib.stream_ptr())
        _lib.check_rc(rc, "cb_peer_copy")
        flag = (ctypes.c_void_p * 1)(self.buf.ptrs[peer] + self.flag_off[kind] + slot * 8)
        rc = lib.cb_signal_peers(flag, 0, 1, 0, ctypes.c_ulonglong(n + 1), _lib.stream_ptr())
        _lib.check_rc(rc, "cb_signal_peers")

    def take(self, kind: str) -> torch.Tensor:
        """Make the stream wait (bounded) for the next message of stream ``kind``; returns it."""
        import ctypes
        from ..ops import _lib
        lib = _lib.lib()
        n = self.taken[kind]
        slot = n % self.depths[kind]
        self.taken[kind] = n + 1
        flag = self.buf.local_ptr + self.flag_off[kind] + slot * 8
        rc = lib.cb_wait_flags(ctypes.c_void_p(flag), 0, 1, ctypes.c_ulonglong(n + 1),
                               ctypes.c_ulonglong(self.limit_ns),
                               _lib.ptr(_lib.status_buffer(self.device)), _lib.stream_ptr())
        _lib.check_rc(rc, "cb_wait_flags")
        off = self.data_off[kind] + slot * self.slot_bytes
        t = self.buf.view(self.dtype, off, self.numel).view(self.shape)
        return t.clone() if self.copy_out else t

    def close(self) -> None:
        self.buf.close()


class _PeerChannel:
    """The interface of :class:`_Channel` over a :class:`PeerRing`."""

    def __init__(self, ring: PeerRing, kind: str, peer: int, recv: bool) -> None:
        self.ring, self.kind, self.peer, self.recv = ring, kind, peer, recv
        self.pending: List = []

    def post_recv(self, force: bool = False) -> None:
        pass

    def take(self) -> torch.Tensor:
        return self.ring.take(self.kind)

    def send(self, t: torch.Tensor) -> None:
        self.ring.push(self.kind, self.peer, t)

    def drain(self) -> None:
        pass


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


def _new_group(ranks, members_only: bool):
    """A process group over ``ranks``.  ``members_only``: only these ranks make the call (several
    pipelines side by side create their groups independently of one another)."""
    if members_only:
        return dist.new_group(ranks, use_local_synchronization=True)
    return dist.new_group(ranks)


def _other_replica_saves(dp_group) -> bool:
    """With replicas of the pipeline the first one writes the checkpoint (all hold the same
    state); the others wait until it is written."""
    if dp_group is None:
        return False
    first = dist.get_rank(dp_group) == 0
    if not first:
        dist.barrier(group=dp_group)
    return not first


def _check_transport(transport: str, device) -> str:
    if transport not in ("nccl", "peer"):
        raise ProcessingError.invalid_input(f"unknown pipeline transport {transport!r}")
    if transport == "peer" and torch.device(device).type != "cuda":
        raise ProcessingError.unsupported("the peer-memory pipeline transport on a CPU rank",
                                          "it moves tensors with NVLink peer stores")
    return transport


def _check_slots(peer_slots: str) -> str:
    if peer_slots not in ("bounded", "message"):
        raise ProcessingError.invalid_input(f"unknown slot policy {peer_slots!r}")
    return peer_slots


def _ring_for(ring: Optional[PeerRing], group, device, shape, dtype, counts, bounded: bool,
              stages: int, micro_batches: int, chunks: int, limit_ms: float = 30000.0) -> PeerRing:
    """The ring that fits these messages: the one at hand, or a new one (every rank of the group
    reaches this at the same step, so the allocation is collective).  ``bounded``: slots for the
    messages that can be on their way at once, copied out on receipt; else a slot per message of
    a step, used in place."""
    want = {k: int(counts.get(k, 0)) for k in PeerRing.KINDS}
    if bounded:
        need = ring_depths(stages, micro_batches, chunks)
        want = {k: min(want[k], need.get(k, 1)) if want[k] else 0 for k in want}
    if ring is not None and ring.shape == tuple(shape) and ring.dtype == dtype \
            and ring.depths == want and ring.copy_out == bounded:
        return ring
    if ring is not None:
        torch.cuda.synchronize(device)
        dist.barrier(group=group)       # nobody still pushes into the buffer that goes away
        ring.close()
    return PeerRing(group, device, shape, dtype, want, limit_ms, copy_out=bounded)


class PipelineStage:
    """One rank's share of a pipelined decoder plus the 1F1B step loop."""

    def __init__(self, cfg: DecoderConfig, group, device, micro_batches: int, seed: int = 0,
                 dtype: torch.dtype = torch.bfloat16, train_cfg=None, schedule=None,
                 transport: str = "nccl", peer_wait_ms: float = 30000.0,
                 peer_slots: str = "bounded", dp_group=None) -> None:
        """``dp_group``: the ranks that hold the same stage in other replicas of the pipeline;
        their gradients are averaged before the optimizer step (every replica is fed its own
        part of the batch)."""
        from ..optim.adamw import AdamW
        from ..train.trainer import TrainConfig
        self.schedule = schedule          # object with at(step) -> learning rate
        self.dp_group = dp_group
        self.dp_size = dist.get_world_size(dp_group) if dp_group is not None else 1
        self.transport = _check_transport(transport, device)
        self._ring: Optional[PeerRing] = None
        self.peer_wait_ms = peer_wait_ms       # bound of one wait for a message, peer transport
        self.peer_slots = _check_slots(peer_slots)
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
            # two groups: traffic of one direction never queues behind the other (with replicas
            # only the members of this pipeline make the call)
            self.fwd_group = _new_group(ranks, dp_group is not None)
            self.bwd_group = _new_group(ranks, dp_group is not None)
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
        if _other_replica_saves(self.dp_group):
            return
        barrier = (lambda: dist.barrier(group=self.group)) if self.stages > 1 else None
        save_named(directory, self.stage, model_state(self.model, self.opt),
                   {"stages": self.stages, "opt_step": self.opt.step_count,
                    "train_step": self.step_index, "config": self.cfg.to_dict()}, barrier)
        if self.dp_group is not None:
            dist.barrier(group=self.dp_group)

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
        chans: Dict[str, object] = {}
        if self.stages > 1 and self.transport == "peer":
            self._ring = _ring_for(self._ring, self.group, self.device, (T, H), act_dtype,
                                   {"f": M, "b": M}, self.peer_slots == "bounded", self.stages, M,
                                   1, self.peer_wait_ms)
            if not self.first:
                chans["rf"] = _PeerChannel(self._ring, "f", self.stage - 1, True)
                chans["sb"] = _PeerChannel(self._ring, "b", self.stage - 1, False)
            if not self.last:
                chans["sf"] = _PeerChannel(self._ring, "f", self.stage + 1, False)
                chans["rb"] = _PeerChannel(self._ring, "b", self.stage + 1, True)
        elif self.stages > 1:
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
                    loss = m.loss_from_hidden(xf, targets[i], save,
                                              grad_scale=1.0 / (T * M * self.dp_size))
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
        if self.dp_group is not None:      # the loss scale already holds 1 / replicas
            dist.all_reduce(m.g32, group=self.dp_group)
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
                 schedule=None, transport: Optional[str] = None,
                 peer_wait_ms: float = 30000.0, peer_slots: str = "bounded",
                 dp_group=None) -> None:
        """``dp_group``: as for :class:`PipelineStage`."""
        from ..optim.adamw import AdamW
        from ..train.trainer import TrainConfig
        self.schedule = schedule
        self.dp_group = dp_group
        self.dp_size = dist.get_world_size(dp_group) if dp_group is not None else 1
        self.group = group
        self.stage = dist.get_rank(group)
        self.stages = dist.get_world_size(group)
        if self.stages < 2 or chunks < 2:
            raise ProcessingError.invalid_input(
                "the interleaved pipeline needs at least two ranks and two chunks per rank")
        on_gpu = torch.device(device).type == "cuda"
        self.transport = _check_transport(transport or ("peer" if on_gpu else "nccl"), device)
        if on_gpu and self.transport == "nccl" \
                and nccl_order_deadlocks(self.stages, micro_batches, chunks):
            raise ProcessingError.unsupported(
                "this interleaved schedule over NCCL point-to-point on GPUs",
                "its order of sends and receives can stop under rendezvous semantics; "
                "use transport='peer'")
        self._ring: Optional[PeerRing] = None
        self.peer_wait_ms = peer_wait_ms
        self.peer_slots = _check_slots(peer_slots)
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
        self._groups = {k: _new_group(ranks, dp_group is not None) for k in ("f", "fw", "b", "bw")}
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
        if _other_replica_saves(self.dp_group):
            return
        save_named(directory, self.stage, self._state(),
                   {"stages": self.stages, "chunks": self.v, "opt_step": self.opts[0].step_count,
                    "train_step": self.step_index, "config": self.cfg.to_dict()},
                   lambda: dist.barrier(group=self.group))
        if self.dp_group is not None:
            dist.barrier(group=self.dp_group)

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

        if self.transport == "peer":
            self._ring = _ring_for(self._ring, self.group, self.device, (T, H), dt,
                                   {"f": M * v, "b": M * v, "fw": n_wrap, "bw": n_wrap},
                                   self.peer_slots == "bounded", P, M, v, self.peer_wait_ms)
            nxt, prv = (s + 1) % P, (s - 1) % P      # group ranks index the ring's peer pointers

        def chan(key, peer, count, recv):
            if self.transport == "peer":
                return _PeerChannel(self._ring, key, peer, recv)
            return _Channel(self._groups[key], peer, (T, H), dt, self.device, count, recv)

        ch: Dict[str, object] = {}
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
                    loss = m.loss_from_hidden(xf, targets[i], save,
                                              grad_scale=1.0 / (T * M * self.dp_size))
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
        if self.dp_group is not None:      # the loss scale already holds 1 / replicas
            for m in self.models:
                dist.all_reduce(m.g32, group=self.dp_group)
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
