"""Expert parallelism for mixture-of-experts feed-forward layers.

Tokens are routed (softmax, top-k, capacity ``C`` per (source rank, expert)), permuted into an
expert-major send buffer and exchanged with the ranks that own the experts; the experts run a
gate/up GEMM, SwiGLU and a down GEMM; results return to the source rank, which sums the ``k``
weighted expert outputs per token.

``backend="fused"``: the exchange happens inside the expert GEMMs (``csrc/gemm.cu``).  The
gate/up GEMM of a local expert pulls that expert's region of every peer's send buffer over
NVLink while it already multiplies the rows that arrived (the all-gather->GEMM kernel with the
peer pointers biased to the expert's region); the down GEMM pushes each finished tile straight
into the source rank's return buffer from its epilogue (the GEMM->reduce-scatter kernel).  No
separate all-to-all runs.  ``backend="nccl"`` uses ``all_to_all_single`` around plain GEMMs: the
baseline, and the path of CPU ranks.  The reference has no experts and no parallelism.
"""
from __future__ import annotations

import ctypes
import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..foundation.error import ProcessingError
from ..ops import _lib
from ..ops import elementwise as E
from ..ops import gemm as G
from ..ops import moe as M
from .tp import _CommArgs


def capacity_for(tokens_per_rank: int, num_experts: int, top_k: int, factor: float) -> int:
    """Rows reserved per (source rank, expert): ``factor * T * k / E`` rounded up to 128."""
    c = int(math.ceil(factor * tokens_per_rank * top_k / num_experts))
    return (c + 127) // 128 * 128


class ExpertParallel:
    """Communication state of one expert-parallel group (buffers are shared by all layers)."""

    def __init__(self, group, device, backend: Optional[str] = None,
                 wait_limit_ms: float = 5000.0) -> None:
        self.group = group
        self.device = torch.device(device)
        self.rank = dist.get_rank(group) if group is not None else 0
        self.ep = dist.get_world_size(group) if group is not None else 1
        if backend is None:
            backend = "fused" if self.device.type == "cuda" and self.ep > 1 else "nccl"
        self.backend = backend
        self.limit_ns = int(wait_limit_ms * 1e6)
        self._bufs: Dict[str, dict] = {}
        self.pad = None
        if backend == "fused":
            from .symm import SignalPad
            self.pad = SignalPad(8, group, self.device, wait_limit_ms)   # 4 slots x {fwd, bwd}

    def buffers(self, tag: str, E_: int, C: int, H: int, dtype) -> dict:
        """``send`` / ``ret`` ``[E*C, H]`` (symmetric when fused), per-direction epoch."""
        key = f"{tag}:{E_}:{C}:{H}"
        b = self._bufs.get(key)
        if b is None:
            b = {"epoch": 0, "slot0": 0 if tag == "f" else 4}
            n = E_ * C * H
            if self.backend == "fused":
                from .symm import SymmetricBuffer
                b["send_sym"] = SymmetricBuffer(n * 2, self.group, self.device)
                b["ret_sym"] = SymmetricBuffer(n * 2, self.group, self.device)
                b["send"] = b["send_sym"].view(torch.bfloat16, 0, n).view(E_ * C, H)
                b["ret"] = b["ret_sym"].view(torch.bfloat16, 0, n).view(E_ * C, H)
                b["flags"] = torch.zeros((E_, (self.ep * C) // 128), dtype=torch.int32,
                                         device=self.device)
            else:
                b["send"] = torch.zeros((E_ * C, H), dtype=dtype, device=self.device)
                b["ret"] = torch.zeros((E_ * C, H), dtype=dtype, device=self.device)
            self._bufs[key] = b
        return b

    # ------------------------------------------------------------------ fused GEMM calls
    def _fused(self, comm: int, a, w, out, C: int, e_global: int, b: dict, j: int, b_mn: bool):
        c = _CommArgs()
        H_bytes = 2
        c.comm, c.tp, c.rank, c.rows_per_shard = comm, self.ep, self.rank, C
        K = a.shape[1]
        N = w.shape[1] if b_mn else w.shape[0]
        if comm == 1:
            width = K
            for s in range(self.ep):
                c.ag_src[s] = b["send_sym"].ptrs[s] + (e_global * C - s * C) * width * H_bytes
            c.ag_flags = b["flags"][j].data_ptr()
            c.ag_epoch = b["epoch"]
            c.peer_flags = self.pad.buf.local_ptr + 8 * b["slot0"] * self.ep
            c.peer_expect = b["epoch"]
        else:
            for s in range(self.ep):
                c.rs_dst[s] = b["ret_sym"].ptrs[s] + e_global * C * N * H_bytes
            c.rs_ld = N
        c.wait_limit_ns = self.limit_ns
        st = _lib.status_buffer(self.device)
        rc = _lib.lib().cb_gemm_bf16_fused(
            _lib.ptr(a), _lib.ptr(w), _lib.ptr(out), a.shape[0], N, K, a.stride(0), w.stride(0),
            out.stride(0) if out is not None else N, int(b_mn), _lib.ptr(None),
            256 if N > 128 else 128, ctypes.byref(c), _lib.ptr(st), 0, _lib.stream_ptr())
        _lib.check_rc(rc, "cb_gemm_bf16_fused(moe)")

    # ------------------------------------------------------------------ exchange + expert FFN
    def run_experts(self, tag: str, b: dict, C: int, El: int, first, second) -> None:
        """Generic two-GEMM expert pass over exchanged rows.

        ``first(j, xg, fused_ag)`` must return the ``[ep*C, K2]`` input of the second GEMM given
        the gathered rows ``xg`` of local expert ``j`` (``fused_ag(w, b_mn, out)`` performs the
        GEMM that pulls the rows from the peers);
        ``second(j, a2)`` returns ``(w2, b_mn)`` for the GEMM whose result rows go back."""
        ep, r = self.ep, self.rank
        send, ret = b["send"], b["ret"]
        H = send.shape[1]
        b["epoch"] += 1
        epoch, s0 = b["epoch"], b["slot0"]
        if self.backend == "fused" and ep > 1:
            self.pad.signal(s0 + 0, epoch)                         # my send buffer is written
            a2s = []
            for j in range(El):
                e = r * El + j
                xg = torch.empty((ep * C, H), dtype=send.dtype, device=self.device)
                xg[r * C:(r + 1) * C].copy_(send[e * C:(e + 1) * C])
                a2s.append(first(j, xg, lambda w, b_mn, out, j=j, e=e, xg=xg:
                                 self._fused(1, xg, w, out, C, e, b, j, b_mn)))
            self.pad.signal(s0 + 1, epoch)                         # I have pulled everything
            if epoch > 1:
                self.pad.wait(s0 + 3, epoch - 1)                   # sources consumed last results
            for j in range(El):
                w2, b_mn = second(j, a2s[j])
                self._fused(2, a2s[j], w2, None, C, r * El + j, b, j, b_mn)
            self.pad.signal(s0 + 2, epoch)                         # results are in your buffers
            self.pad.wait(s0 + 2, epoch)                           # ... and theirs are in mine
            return
        raise ProcessingError.invalid_input(
            "run_experts is the fused transport; use run_experts_grouped with this backend")

    @property
    def fused(self) -> bool:
        return self.backend == "fused" and self.ep > 1

    def run_experts_grouped(self, b: dict, C: int, El: int, first_all, second_all) -> None:
        """The same two-GEMM pass with a library all-to-all (or none on one rank) around grouped
        GEMMs: ``first_all(xg)`` maps the exchanged rows ``[El, ep*C, H]`` of all local experts to
        the input ``[El, ep*C, K2]`` of the second GEMM; ``second_all()`` returns the stacked
        weights ``(w2, b_mn)`` of the GEMM whose result rows go back."""
        ep = self.ep
        send, ret = b["send"], b["ret"]
        H = send.shape[1]
        b["epoch"] += 1
        if ep > 1:
            recv = torch.empty_like(send)
            dist.all_to_all_single(recv, send, group=self.group)    # [ep(src), El, C, H]
            xg = recv.view(ep, El, C, H).permute(1, 0, 2, 3).reshape(El, ep * C, H)
        else:
            # a private copy: the send buffer is reused by the next layer while backward needs
            # these rows
            xg = send.view(El, C, H).clone()
        a2 = first_all(xg)
        w2, b_mn = second_all()
        if ep > 1:
            out = G.gemm_grouped(a2, w2, b_mn=b_mn)                 # [El, ep*C, H]
            back = out.view(El, ep, C, -1).permute(1, 0, 2, 3).contiguous()
            dist.all_to_all_single(ret.view(ep, El, C, -1), back, group=self.group)
        else:
            G.gemm_grouped(a2, w2, b_mn=b_mn, out=ret.view(El, C, -1))

    def before_send_write(self, b: dict) -> None:
        if self.backend == "fused" and self.ep > 1 and b["epoch"] > 0:
            self.pad.wait(b["slot0"] + 1, b["epoch"])              # everyone pulled my last send

    def after_combine(self, b: dict) -> None:
        if self.backend == "fused" and self.ep > 1:
            self.pad.signal(b["slot0"] + 3, b["epoch"])


class MoEFFN:
    """One mixture-of-experts feed-forward layer: router ``[H, E]`` (replicated), local experts'
    ``gate_up [El, H, 2I]`` and ``down [El, I, H]``.  Weights live in fp32 masters with a working
    copy in the activation dtype; gradients accumulate in fp32."""

    def __init__(self, hidden: int, inter: int, num_experts: int, top_k: int,
                 capacity_factor: float, epx: ExpertParallel, aux_coef: float = 0.01,
                 init_std: float = 0.02, seed: int = 0, dtype=torch.bfloat16,
                 allocate: bool = True) -> None:
        if num_experts % epx.ep:
            raise ProcessingError.invalid_input("num_experts must be divisible by the EP degree")
        self.H, self.I, self.E, self.k = hidden, inter, num_experts, top_k
        self.cf, self.epx, self.aux_coef = capacity_factor, epx, aux_coef
        self.El = num_experts // epx.ep
        dev = epx.device
        self.dtype = dtype
        self._saved = None
        self.last_aux = None
        self.master, self.w, self.g = {}, {}, {}
        if not allocate:        # the owner binds views of its flat buffers
            return
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed)                       # router: same on every rank
        self.master = {"router": torch.empty(hidden, num_experts, device=dev).normal_(0, init_std, generator=gen)}
        gen.manual_seed(seed * 7919 + 1 + epx.rank)  # experts: rank specific
        self.master["gate_up"] = torch.empty(self.El, hidden, 2 * inter, device=dev).normal_(0, init_std, generator=gen)
        self.master["down"] = torch.empty(self.El, inter, hidden, device=dev).normal_(0, init_std, generator=gen)
        self.w = {k: v.to(dtype) for k, v in self.master.items()}
        self.g = {k: torch.zeros_like(v) for k, v in self.master.items()}

    def routing_stats(self) -> dict:
        """Load per expert and dropped share of the last forward pass (host numbers)."""
        if getattr(self, "last_load", None) is None:
            return {}
        load = self.last_load.detach().float().cpu()
        return {"load": load.tolist(), "max_over_mean": float(load.max() * self.E),
                "dropped": float(self.last_dropped)}

    def bind(self, w: dict, g: dict, master: dict) -> None:
        """Use externally owned tensors (keys ``router``, ``gate_up``, ``down``)."""
        self.w, self.g, self.master = w, g, master

    def sync_working_copy(self) -> None:
        for k, v in self.master.items():
            self.w[k].copy_(v)

    def zero_grad(self) -> None:
        for v in self.g.values():
            v.zero_()

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor, resid: Optional[torch.Tensor] = None,
                save: bool = True) -> torch.Tensor:
        """``x [T, H]`` (already normalised); returns ``resid + moe(x)``."""
        epx = self.epx
        T = x.shape[0]
        C = capacity_for(T, self.E, self.k, self.cf)
        if self.E % 8:      # the GEMM kernel wants 16-byte rows; tiny routers take the library path
            logits = x.float() @ self.w["router"].float()
        else:
            logits = G.gemm(x, self.w["router"], b_mn=True, out_dtype=torch.float32)
        expert, w, probs, slot, counts = M.route(logits, self.k, C)
        b = epx.buffers("f", self.E, C, self.H, x.dtype)
        epx.before_send_write(b)
        b["send"].zero_()
        M.gather_rows(x, expert, slot, b["send"], C)
        kept = {}

        def first(j, xg, fused_ag):     # fused transport: the GEMM pulls the rows of expert j
            gu = torch.empty((xg.shape[0], 2 * self.I), dtype=xg.dtype, device=xg.device)
            fused_ag(self.w["gate_up"][j], True, gu)
            act = E.swiglu_fwd(gu)
            kept[j] = (xg, gu, act)
            return act

        def first_all(xg):      # all local experts in one grouped launch per GEMM
            gu = G.gemm_grouped(xg, self.w["gate_up"], b_mn=True)
            act = E.swiglu_fwd(gu.view(-1, 2 * self.I)).view(self.El, -1, self.I)
            kept["all"] = (xg, gu, act)
            return act

        if epx.fused:
            epx.run_experts("f", b, C, self.El, first, lambda j, a2: (self.w["down"][j], True))
        else:
            epx.run_experts_grouped(b, C, self.El, first_all, lambda: (self.w["down"], True))
        out = M.combine_rows(b["ret"], expert, slot, C, w, resid)
        # load-balancing auxiliary loss: E * sum_e f_e * P_e
        frac = torch.zeros(self.E, dtype=torch.float32, device=x.device)
        frac.index_add_(0, expert.reshape(-1).long(), torch.ones(T * self.k, device=x.device))
        frac /= float(T * self.k)
        self.last_aux = self.aux_coef * self.E * (frac * probs.mean(0)).sum()
        # monitoring (device tensors, read on demand): share of the assignments each expert got
        # and share that found no capacity slot
        self.last_load = frac
        self.last_dropped = (slot < 0).float().mean()
        if save:
            self._saved = dict(x=x, expert=expert, w=w, probs=probs, slot=slot, C=C, frac=frac,
                               ret=b["ret"].clone(), kept=kept)
        epx.after_combine(b)
        return out

    # ------------------------------------------------------------------ backward
    def backward(self, dout: torch.Tensor, aux_grad_scale: float = 1.0) -> torch.Tensor:
        """Gradient w.r.t. the layer input ``x`` (the residual path is the caller's).
        ``aux_grad_scale`` multiplies the gradient of the load-balancing term."""
        sv, epx = self._saved, self.epx
        x, expert, w, probs, slot, C = sv["x"], sv["expert"], sv["w"], sv["probs"], sv["slot"], sv["C"]
        T = x.shape[0]
        dw = M.pair_dot(dout, sv["ret"], expert, slot, C)                     # [T, k]
        b = epx.buffers("b", self.E, C, self.H, x.dtype)
        epx.before_send_write(b)
        b["send"].zero_()
        M.gather_rows(dout, expert, slot, b["send"], C, scale=w)
        kept = sv["kept"]

        def first(j, dyg, fused_ag):
            xg, gu, act = kept[j]
            dact = torch.empty((dyg.shape[0], self.I), dtype=dyg.dtype, device=dyg.device)
            fused_ag(self.w["down"][j], False, dact)
            G.linear_wgrad(act, dyg, self.g["down"][j])
            dgu = E.swiglu_bwd(gu, dact)
            G.linear_wgrad(xg, dgu, self.g["gate_up"][j])
            return dgu

        def first_all(dyg):
            xg, gu, act = kept["all"]
            dact = G.gemm_grouped(dyg, self.w["down"], b_mn=False)
            G.linear_wgrad_grouped(act, dyg, self.g["down"])
            dgu = E.swiglu_bwd(gu.view(-1, 2 * self.I), dact.view(-1, self.I)).view(
                self.El, -1, 2 * self.I)
            G.linear_wgrad_grouped(xg, dgu, self.g["gate_up"])
            return dgu

        if epx.fused:
            epx.run_experts("b", b, C, self.El, first,
                            lambda j, a2: (self.w["gate_up"][j], False))
        else:
            epx.run_experts_grouped(b, C, self.El, first_all,
                                    lambda: (self.w["gate_up"], False))
        dx = M.combine_rows(b["ret"], expert, slot, C, None, None)
        epx.after_combine(b)
        # router: w_k = p_k / sum_j p_j over the chosen experts, plus the auxiliary loss
        idx = expert.long()
        pk = probs.gather(1, idx)
        s = pk.sum(-1, keepdim=True)
        dpk = (dw - (dw * w).sum(-1, keepdim=True)) / s
        dprobs = torch.zeros_like(probs).scatter_add_(1, idx, dpk)
        dprobs += (aux_grad_scale * self.aux_coef * self.E / T) * sv["frac"][None, :]
        dlogits = probs * (dprobs - (dprobs * probs).sum(-1, keepdim=True))
        dl = dlogits.to(x.dtype)
        if not x.is_cuda or self.E % 8:
            self.g["router"] += x.float().t() @ dlogits
            dx_r = (dlogits @ self.w["router"].float().t()).to(x.dtype)
        else:
            G.gemm(x, dl, a_mn=True, b_mn=True, out=self.g["router"], accumulate=True)
            dx_r = G.gemm(dl, self.w["router"], b_mn=False)
        self._saved = None
        return (dx.float() + dx_r.float()).to(x.dtype)


def dense_spans(layout) -> List[Tuple[int, int]]:
    """Maximal ``[start, end)`` ranges of the flat buffers that hold no expert weights (these are
    replicated over the expert-parallel group and need the gradient all-reduce)."""
    spans, start = [], 0
    for s in sorted(layout.specs, key=lambda s: s.offset):
        if s.expert:
            if s.offset > start:
                spans.append((start, s.offset))
            a = layout.ALIGN
            start = s.offset + (s.numel + a - 1) // a * a
    if layout.total > start:
        spans.append((start, layout.total))
    return spans


class ExpertParallelTrainer:
    """Training step of a mixture-of-experts decoder whose expert-parallel group is also its
    data-parallel group: every rank runs its own tokens, expert weights are owned by one rank
    (their gradients are complete once the exchanged rows have been processed), all other
    gradients are summed over the group while backward is still running."""

    def __init__(self, model, cfg=None, overlap: bool = True, schedule=None) -> None:
        """``overlap=False`` runs the dense all-reduces after the backward pass instead of
        concurrently with it (no collective kernel then shares the SMs with expert GEMMs that
        wait on peers)."""
        from ..optim.adamw import AdamW
        self.overlap = overlap
        self.schedule = schedule          # object with at(step) -> learning rate
        from ..train.trainer import TrainConfig
        self.model, self.cfg = model, cfg or TrainConfig()
        self.epx: ExpertParallel = model.epx
        self.opt = AdamW(self.cfg.adamw(), 0, model.n_flat, model.layout.decay_end, model.device)
        self.spans = dense_spans(model.layout)
        L = model.cfg.num_layers
        if len(self.spans) != L + 1:
            raise ProcessingError.invalid_input("unexpected parameter layout for expert parallelism")
        # the last span holds the LM head (complete after the head's backward) and the vectors
        # (complete at the very end)
        lo, hi = self.spans[-1]
        d = min(max(model.layout.decay_end, lo), hi)
        self._head, self._tail = (lo, d), (d, hi)
        self.step_index = 0
        self._stream = torch.cuda.Stream(model.device) if model.device.type == "cuda" else None
        if self.epx.ep > 1:
            # global gradient norm: the dense gradients are already summed over the group and equal
            # on every rank, the expert gradients exist on one rank each
            def norm_hook(g32, sumsq):
                dense = torch.zeros_like(sumsq)
                for lo_, hi_ in self.spans:
                    if hi_ > lo_:
                        E.sumsq_into(g32[lo_:hi_], dense)
                experts = sumsq - dense
                dist.all_reduce(experts, group=self.epx.group)
                sumsq.copy_(experts + dense)
            self.opt.norm_hook = norm_hook

    def _reduce(self, span: Tuple[int, int]) -> None:
        if self.epx.ep == 1 or span[1] <= span[0]:
            return
        g = self.model.g32[span[0]:span[1]]
        if self._stream is None:
            dist.all_reduce(g, group=self.epx.group)
            return
        self._stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self._stream):
            dist.all_reduce(g, group=self.epx.group)

    def _on_layer_done(self, l: int) -> None:
        if not self.overlap:
            return
        if l == -1:
            self._reduce(self._head)
        elif l >= 1:
            self._reduce(self.spans[l])     # attention + router weights of layer l
        # l == 0 and l == -2: the first span also holds the embedding; it goes last

    def save_checkpoint(self, directory: str) -> None:
        """Name-keyed training checkpoint: rank 0's file holds the replicated tensors and its
        experts, the other ranks' files their experts (with the replicated tensors again, which
        a loader takes from the first file that has them); loads into any expert-parallel
        degree."""
        from ..checkpoint.named import model_state, save_named
        barrier = (lambda: dist.barrier(group=self.epx.group)) if self.epx.ep > 1 else None
        save_named(directory, self.epx.rank, model_state(self.model, self.opt),
                   {"ep": self.epx.ep, "opt_step": self.opt.step_count,
                    "train_step": getattr(self, "step_index", 0),
                    "config": self.model.cfg.to_dict()}, barrier)

    def load_checkpoint(self, directory: str) -> dict:
        from ..checkpoint.named import load_named, model_state
        man = load_named(directory, model_state(self.model, self.opt))
        self.model.sync_working_copy()
        self.opt.step_count = int(man["opt_step"])
        self.step_index = int(man["train_step"])
        return man

    def train_step(self, ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        m, ep = self.model, self.epx.ep
        T = ids.numel()
        if self.schedule is not None:
            self.opt.set_learning_rate(self.schedule.at(self.step_index))
        m.zero_grad()
        loss = m.forward_loss(ids, targets, grad_scale=1.0 / (T * ep))
        m.backward(on_layer_done=self._on_layer_done)
        if not self.overlap:
            self._reduce(self._head)
            for span in self.spans[1:-1]:
                self._reduce(span)
        self._reduce(self.spans[0])
        self._reduce(self._tail)
        if self._stream is not None:
            torch.cuda.current_stream().wait_stream(self._stream)
        self.opt.step(m.p32, m.g32, m.p16, 1.0)
        self.step_index += 1
        return loss
