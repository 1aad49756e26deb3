"""Sharded data parallelism (optimizer state and master-weight updates sharded 1/N).

Each rank computes full gradients for its own micro-batch into its fp32 flat gradient buffer.
The flat buffer is cut into buckets that follow the backward pass (``plans.build_buckets``); as
soon as a bucket's gradients are complete on a rank, that rank signals its peers, and the owner
of each shard of the bucket runs ONE kernel (``csrc/comm.cu: rs_adamw_ag_kernel``) that

* reads the shard from every rank's gradient buffer over NVLink (the reduce-scatter): with
  ``multimem.ld_reduce`` through an NVLink multicast mapping where the devices have one (the sum
  is formed in the switch), else with plain peer loads added in rank order,
* scales it and applies AdamW to its fp32 master weights and moments,
* writes the new bf16 weights into every rank's working copy (the all-gather): one
  ``multimem.st``, or a store per rank,

on a side stream, overlapped with the rest of the backward pass.  ``backend="collective"`` does
the same arithmetic with ``torch.distributed`` collectives (reduce-scatter / all-gather on NCCL,
all-reduce on Gloo); it is the baseline the fused kernel is measured against, the path used on
CPU ranks, and the fallback when peer mapping is unavailable.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch
import torch.distributed as dist

from ..foundation.error import ProcessingError
from ..ops import _lib
from ..ops import elementwise as E
from ..optim.adamw import AdamWConfig
from .plans import Bucket, build_buckets, moment_offsets


class _ShardedOptState:
    def __init__(self, n: int, device) -> None:
        self.m = torch.zeros(n, dtype=torch.float32, device=device)
        self.v = torch.zeros(n, dtype=torch.float32, device=device)
        self.step_count = 0

    def state_dict(self):
        return {"m": self.m, "v": self.v, "step": self.step_count}

    def load_state_dict(self, sd):
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        self.step_count = int(sd["step"])


class ShardedDataParallel:
    def __init__(self, group, device, backend: Optional[str] = None,
                 comm_blocks: Optional[int] = None, wait_limit_ms: float = 5000.0,
                 tail_blocks: Optional[int] = None, nvls: Optional[bool] = None) -> None:
        """``comm_blocks``: thread blocks (of 128 threads) of a bucket kernel that runs beside the
        backward pass: about one per SM, small enough to share the SM with a persistent compute
        CTA; ``tail_blocks``: blocks of the buckets that complete when the backward pass ends and
        have nothing left to hide behind."""
        self.group = group
        self.device = torch.device(device)
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if backend is None:
            backend = "p2p" if self.device.type == "cuda" else "collective"
        if backend not in ("p2p", "collective"):
            raise ProcessingError.invalid_input(f"unknown data-parallel backend '{backend}'")
        self.backend = backend
        if comm_blocks is None:
            comm_blocks = int(os.environ.get("COEUS_DP_BLOCKS", "128"))
        if tail_blocks is None:
            tail_blocks = int(os.environ.get("COEUS_DP_TAIL_BLOCKS", "592"))
        self.comm_blocks, self.tail_blocks = comm_blocks, tail_blocks
        self.nvls = (os.environ.get("COEUS_DP_NVLS", "0") == "1") if nvls is None else bool(nvls)
        self.wait_limit_ms = wait_limit_ms
        self.model = None

    # ------------------------------------------------------------------ set-up
    def attach(self, model, opt_cfg: AdamWConfig) -> None:
        self.model = model
        model.dropout_rank = self.rank      # replicas draw different dropout masks
        self.opt_cfg = opt_cfg
        self.buckets: List[Bucket] = build_buckets(model.layout, model.n_flat)
        self.moffs, mtotal = moment_offsets(self.buckets, self.rank, self.world)
        self.opt = _ShardedOptState(mtotal, self.device)
        self.by_trigger = {}
        for b in self.buckets:
            self.by_trigger.setdefault(b.trigger, []).append(b)
        self.step_no = 0
        # all replicas start from rank 0's weights
        dist.broadcast(model.p32, src=dist.get_global_rank(self.group, 0), group=self.group)
        model.sync_working_copy()
        if self.backend == "p2p":
            from .symm import MulticastBuffer, SignalPad, SymmetricBuffer, multicast_supported
            n = model.n_flat
            # Gradient and weight buffers: symmetric memory bound to an NVLink multicast object
            # where the devices support it (the bucket kernel then reduces in the switch with
            # multimem.ld_reduce and broadcasts with multimem.st), plain peer mappings otherwise.
            # All ranks must take the same branch, hence the agreement over the group.
            self.g_mc = self.p_mc = None
            # (measured on 8 B200s the two paths are within noise of each other over a whole
            # step -- 41.4 against 41.5 ms -- and at two ranks the plain path is ahead, so the
            # multicast path is opt-in: nvls=True or COEUS_DP_NVLS=1)
            want = self.world > 1 and self.nvls and multicast_supported(self.device)
            ok = torch.tensor([1 if want else 0], device=self.device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
            if int(ok) == 1:
                try:
                    self.sym_g = MulticastBuffer(n * 4, self.group, self.device)
                    self.sym_p = MulticastBuffer(n * 2, self.group, self.device)
                    self.g_mc, self.p_mc = self.sym_g.mc_ptr, self.sym_p.mc_ptr
                    if os.environ.get("COEUS_DP_MC_KERNEL", "1") == "0":
                        # tuning aid: multicast-bound buffers, plain peer loads in the kernel
                        self.g_mc = self.p_mc = 0
                except Exception:
                    ok.fill_(0)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
                if int(ok) == 0:        # some rank failed: everybody falls back together
                    for b in (getattr(self, "sym_g", None), getattr(self, "sym_p", None)):
                        if isinstance(b, MulticastBuffer):
                            b.close()
                    self.g_mc = self.p_mc = None
            if self.g_mc == 0:
                self.g_mc = self.p_mc = None
            elif self.g_mc is None:
                self.sym_g = SymmetricBuffer(n * 4, self.group, self.device)
                self.sym_p = SymmetricBuffer(n * 2, self.group, self.device)
            model.rebind(p16=self.sym_p.view(torch.bfloat16, 0, n),
                         g32=self.sym_g.view(torch.float32, 0, n))
            self.pad = SignalPad(len(self.buckets) + 1, self.group, self.device,
                                 self.wait_limit_ms)
            self.g_ptrs = self.sym_g.ptr_array()
            self.p_ptrs = self.sym_p.ptr_array()
            self.flag_ptrs = self.pad.buf.ptr_array()
            self.comm_stream = torch.cuda.Stream(
                device=self.device, priority=int(os.environ.get("COEUS_DP_PRIORITY", "-1")))
            self.events = [torch.cuda.Event() for _ in self.buckets]
            self.done_event = torch.cuda.Event()
            # gradient clipping: per-bucket, per-block sums of squares of the reduced shards
            self._slots = max(self.comm_blocks, self.tail_blocks, 64)
            self.partials = torch.zeros(len(self.buckets) * self._slots, dtype=torch.float32,
                                        device=self.device)
            self.clip_coef = torch.ones(1, dtype=torch.float32, device=self.device)
            self.grad_norm = torch.zeros(1, dtype=torch.float32, device=self.device)
            dist.barrier(group=self.group)

    # ------------------------------------------------------------------ step protocol
    def begin_step(self) -> None:
        """Before gradients are zeroed and weights are read: every rank must have finished
        reading our gradients and writing our weights in the previous step."""
        self.step_no += 1
        if self.backend == "p2p" and self.step_no > 1:
            torch.cuda.current_stream().wait_event(self.done_event)
            self.pad.wait(len(self.buckets), self.step_no - 1)

    def on_layer_done(self, trigger: int) -> None:
        if self.backend != "p2p":
            return
        for b in self.by_trigger.get(trigger, []):
            self._launch_bucket(b)

    def _bucket_kernel(self, b: Bucket, mode: int) -> None:
        """``mode`` 0: reduce-scatter + AdamW + all-gather; 1: reduce-scatter + sum of squares;
        2: AdamW (gradients times the clip coefficient) + all-gather."""
        c = self.opt_cfg
        # buckets completed by the end of the backward pass (and the second pass of a clipped
        # step) run alone: they take the whole machine
        blocks = self.tail_blocks if (b.trigger == -2 or mode == 2) else self.comm_blocks
        s, e = b.shard(self.rank, self.world)
        m = self.model
        st = _lib.status_buffer(self.device)
        part = self.partials[b.index * self._slots:]
        rc = _lib.lib().cb_rs_adamw_ag(
            self.g_ptrs, self.p_ptrs, _lib.ptr(m.p32), _lib.ptr(self.opt.m),
            _lib.ptr(self.opt.v), ctypes.c_size_t(s), ctypes.c_size_t(e),
            ctypes.c_size_t(self.moffs[b.index]), ctypes.c_size_t(m.layout.decay_end),
            ctypes.c_float(c.lr), ctypes.c_float(c.beta1), ctypes.c_float(c.beta2),
            ctypes.c_float(c.eps), ctypes.c_float(c.weight_decay), self.step_no,
            ctypes.c_float(self._grad_scale), self.world,
            ctypes.c_void_p(self.pad.buf.local_ptr), b.index,
            ctypes.c_ulonglong(self.step_no), ctypes.c_ulonglong(self.pad.limit_ns),
            blocks, _lib.ptr(st), _lib.stream_ptr(), mode, self.rank, _lib.ptr(part),
            _lib.ptr(self.clip_coef), ctypes.c_void_p(self.g_mc), ctypes.c_void_p(self.p_mc))
        _lib.check_rc(rc, "cb_rs_adamw_ag")

    def _launch_bucket(self, b: Bucket) -> None:
        ev = self.events[b.index]
        ev.record(torch.cuda.current_stream())
        s, e = b.shard(self.rank, self.world)
        clip = self.opt_cfg.grad_clip is not None
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(ev)
            self.pad.signal(b.index, self.step_no)
            if e > s or clip:
                self._bucket_kernel(b, 1 if clip else 0)

    _grad_scale = 1.0

    def set_grad_scale(self, s: float) -> None:
        self._grad_scale = s

    def reduce_and_step(self, grad_scale: float) -> None:
        """Called after ``backward``.  With the fused backend the bucket kernels were already
        queued by ``on_layer_done``; this only closes the step.  The collective backend does the
        whole reduction and update here."""
        self.opt.step_count += 1
        if self.backend == "p2p":
            with torch.cuda.stream(self.comm_stream):
                if self.opt_cfg.grad_clip is not None:
                    # every bucket has been reduced into its owner's gradient buffer: the global
                    # norm is the root of the sum over owners, then the update runs per bucket
                    sumsq = self.partials.sum().reshape(1)
                    if self.world > 1:
                        dist.all_reduce(sumsq, group=self.group)
                    E.clip_coef_from_sumsq(sumsq, self._grad_scale, self.opt_cfg.grad_clip,
                                           self.clip_coef, self.grad_norm)
                    for b in self.buckets:
                        s, e = b.shard(self.rank, self.world)
                        if e > s:
                            self._bucket_kernel(b, 2)
                self.pad.signal(len(self.buckets), self.step_no)
                self.done_event.record(self.comm_stream)
            return
        m, c = self.model, self.opt_cfg
        coef = None
        if c.grad_clip is not None:
            dist.all_reduce(m.g32, group=self.group)
            sumsq = torch.zeros(1, dtype=torch.float32, device=self.device)
            E.sumsq_into(m.g32, sumsq)
            coef = torch.ones(1, dtype=torch.float32, device=self.device)
            E.clip_coef_from_sumsq(sumsq, grad_scale, c.grad_clip, coef)
            reduced = True
        else:
            reduced = False
        fast = self.device.type == "cuda"
        for b in self.buckets:
            s, e = b.shard(self.rank, self.world)
            equal = (b.end - b.start) % (self.world * 8) == 0
            if not reduced:
                if fast and equal:
                    dist.reduce_scatter_tensor(m.g32[s:e], m.g32[b.start:b.end], group=self.group)
                else:
                    dist.all_reduce(m.g32[b.start:b.end], group=self.group)
            if e > s:
                for lo, hi, wd in ((s, min(e, m.layout.decay_end), c.weight_decay),
                                   (max(s, m.layout.decay_end), e, 0.0)):
                    if hi > lo:
                        mo = self.moffs[b.index] + (lo - s)
                        E.adamw_step(m.p32[lo:hi], self.opt.m[mo:mo + hi - lo],
                                     self.opt.v[mo:mo + hi - lo], m.g32[lo:hi], m.p16[lo:hi],
                                     lr=c.lr, beta1=c.beta1, beta2=c.beta2, eps=c.eps,
                                     weight_decay=wd, step=self.opt.step_count,
                                     grad_scale=grad_scale, clip_coef=coef)
            # all-gather of the updated bf16 shards
            if fast and equal:
                dist.all_gather_into_tensor(m.p16[b.start:b.end], m.p16[s:e], group=self.group)
            else:
                for r in range(self.world):
                    rs, re_ = b.shard(r, self.world)
                    if re_ > rs:
                        dist.broadcast(m.p16[rs:re_], src=dist.get_global_rank(self.group, r),
                                       group=self.group)

    def finish(self) -> None:
        """Drain the side stream (end of training or before checkpointing)."""
        if self.backend == "p2p":
            torch.cuda.current_stream().wait_event(self.done_event)
            self.pad.wait(len(self.buckets), self.step_no)

    def gather_master(self) -> torch.Tensor:
        """Full fp32 master weights assembled from the owners' shards (checkpointing)."""
        self.finish()
        m = self.model
        full = m.p32.clone()
        for b in self.buckets:
            for r in range(self.world):
                s, e = b.shard(r, self.world)
                if e > s:
                    dist.broadcast(full[s:e], src=dist.get_global_rank(self.group, r),
                                   group=self.group)
        return full
