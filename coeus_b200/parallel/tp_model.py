"""Tensor-parallel decoder (Megatron column/row split with sequence-parallel activations).

Per layer: ``norm -> [all-gather -> QKV GEMM] -> attention over the local heads ->
[O GEMM -> reduce-scatter] + residual -> norm -> [all-gather -> gate/up GEMM] -> SwiGLU/GELU ->
[down GEMM -> reduce-scatter] + residual``.  The bracketed pairs are the fused kernels of
:class:`coeus_b200.parallel.tp.TensorParallel`; activations between blocks stay sharded by token
(``[T/tp, H]``).  The LM head is vocabulary-parallel and the loss exchanges only per-token
``(max, sum-exp, target logit)`` triples.  The backward pass mirrors the forward with the two
kernels swapped.  Weights keep the ``[in, out]`` layout; QKV / gate-up are split along ``out``,
O / down along ``in``, the embedding table is replicated.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..foundation.error import ProcessingError
from ..models.config import DecoderConfig
from ..ops import attention as A
from ..ops import elementwise as E
from ..ops import gemm as G
from ..ops import norm as N
from .tp import TensorParallel


class TPDecoderLM:
    def __init__(self, cfg: DecoderConfig, tp: TensorParallel, device, seed: int = 0,
                 dtype: torch.dtype = torch.bfloat16, full=None, recompute: bool = False) -> None:
        """``recompute=True`` keeps only each block's (sequence-sharded) input and runs the
        block's forward, collectives included, again in the backward pass."""
        cfg.validate()
        cfg.require_no_dropout("tensor parallelism")
        self.recompute = bool(recompute)
        if cfg.pos == "learned":
            raise ProcessingError.unsupported(
                "learned positions under tensor parallelism",
                "rotary or sinusoidal positions only there")
        if cfg.use_bias or cfg.num_experts or cfg.tie_embeddings:
            raise ProcessingError.unsupported(
                "tensor-parallel decoder with biases, experts or tied embeddings",
                "use use_bias=False, num_experts=0, tie_embeddings=False")
        n = tp.tp
        if cfg.num_heads % n or cfg.kv_heads % n or cfg.intermediate_dim % (8 * n) \
                or cfg.vocab_padded % (8 * n):
            raise ProcessingError.invalid_input(
                "heads, key/value heads, intermediate_dim/8 and padded vocab/8 must be divisible "
                "by the tensor-parallel degree")
        self.cfg, self.tp, self.device = cfg, tp, torch.device(device)
        self.rank, self.n = tp.rank, n
        H, I, L = cfg.hidden_dim, cfg.intermediate_dim, cfg.num_layers
        self.Hl, self.Il, self.Vl = H // n, I // n, cfg.vocab_padded // n
        self.nh_l = cfg.num_heads // n
        # grouped-query attention: a rank holds whole groups (its query heads and the K/V heads
        # they read), so attention stays local to the rank
        self.kvh_l = cfg.kv_heads // n
        self.Kl = self.kvh_l * cfg.head_dim
        self.gqa = cfg.kv_heads != cfg.num_heads
        self.swiglu = cfg.activation == "swiglu"
        self.rms = cfg.norm == "rmsnorm"
        up_w = 2 * self.Il if self.swiglu else self.Il
        specs: List[Tuple[str, Tuple[int, ...], bool]] = [("token_embed", (cfg.vocab_size, H), True)]
        for l in range(L):
            p = f"layers.{l}."
            specs += [(p + "attn.qkv_weights", (H, self.Hl + 2 * self.Kl), True),
                      (p + "attn.o_weights", (self.Hl, H), True),
                      (p + "ff.up_weights", (H, up_w), True),
                      (p + "ff.down_weights", (self.Il, H), True)]
        specs.append(("output_proj", (H, self.Vl), True))
        self.decay_specs = len(specs)
        for l in range(L):
            p = f"layers.{l}."
            specs.append((p + "norm1_scale", (H,), False))
            if not self.rms:
                specs.append((p + "norm1_bias", (H,), False))
            specs.append((p + "norm2_scale", (H,), False))
            if not self.rms:
                specs.append((p + "norm2_bias", (H,), False))
        specs.append(("final_norm_scale", (H,), False))
        if not self.rms:
            specs.append(("final_norm_bias", (H,), False))
        self.specs = specs
        off, self.offsets = 0, {}
        for i, (name, shape, _) in enumerate(specs):
            self.offsets[name] = (off, shape)
            off += (math.prod(shape) + 63) // 64 * 64
            if i == self.decay_specs - 1:
                self.decay_end = off
        self.n_flat = (off + 1023) // 1024 * 1024
        self.p32 = torch.zeros(self.n_flat, dtype=torch.float32, device=self.device)
        self.p16 = torch.zeros(self.n_flat, dtype=dtype, device=self.device)
        self.g32 = torch.zeros(self.n_flat, dtype=torch.float32, device=self.device)
        self.w, self.g, self.master = {}, {}, {}
        for name, (o, shape) in self.offsets.items():
            k = math.prod(shape)
            self.w[name] = self.p16[o:o + k].view(shape)
            self.g[name] = self.g32[o:o + k].view(shape)
            self.master[name] = self.p32[o:o + k].view(shape)
        self.replicated = ["token_embed"] + [nme for nme, _, d in specs if not d]
        self._pe = None
        self._saved = None
        if full is not None:
            self.load_from_full(full)
        else:
            self._init_like_unsharded(seed)

    # ------------------------------------------------------------------ parameters
    def load_from_full(self, full) -> None:
        """Take this rank's shards out of an unsharded :class:`DecoderLM` with the same config."""
        self._take_shards(lambda name: full.master[name], full.layout.norm_names)

    def _init_like_unsharded(self, seed: int) -> None:
        """Random init that does not depend on the tensor-parallel degree: every tensor is drawn
        whole, with the stream the unsharded model uses for it (one generator seed per tensor
        name), and this rank keeps its slice.  One full tensor lives at a time."""
        import zlib

        from ..models.decoder import ParamLayout
        cfg = self.cfg
        layout = ParamLayout(cfg)
        gen = torch.Generator(device=self.device)

        def draw(name: str) -> torch.Tensor:
            s = layout.by_name[name]
            t = torch.zeros(tuple(s.shape), dtype=torch.float32, device=self.device)
            if s.kind in ("weight", "embed"):
                gen.manual_seed(seed * 1000003 + zlib.crc32(name.encode()))
                t.normal_(0.0, cfg.init_std, generator=gen)
                if name == "output_proj":          # padding columns of the vocabulary stay zero
                    t[:, cfg.vocab_size:].zero_()
            elif s.kind == "scale":
                t.fill_(1.0)
            return t

        self._take_shards(draw, layout.norm_names)

    def _take_shards(self, get, norm_names) -> None:
        """``get(name)`` returns the unsharded fp32 tensor ``name`` (DecoderLM naming)."""
        cfg, r = self.cfg, self.rank
        H, I = cfg.hidden_dim, cfg.intermediate_dim
        Hl, Il, Vl = self.Hl, self.Il, self.Vl
        n1, n2, fn = norm_names
        self.master["token_embed"].copy_(get("token_embed")[:cfg.vocab_size])
        for l in range(cfg.num_layers):
            p = f"layers.{l}."
            wq = get(p + "attn.qkv_weights")
            Kl, Hkv = self.Kl, cfg.kv_dim
            parts = [wq[:, r * Hl:(r + 1) * Hl], wq[:, H + r * Kl:H + (r + 1) * Kl],
                     wq[:, H + Hkv + r * Kl:H + Hkv + (r + 1) * Kl]]
            self.master[p + "attn.qkv_weights"].copy_(torch.cat(parts, 1))
            self.master[p + "attn.o_weights"].copy_(get(p + "attn.o_weights")[r * Hl:(r + 1) * Hl])
            if self.swiglu:
                wg = get(p + "ff.gate_up_weights")
                self.master[p + "ff.up_weights"].copy_(torch.cat(
                    [wg[:, r * Il:(r + 1) * Il], wg[:, I + r * Il:I + (r + 1) * Il]], 1))
            else:
                self.master[p + "ff.up_weights"].copy_(
                    get(p + "ff.up_weights")[:, r * Il:(r + 1) * Il])
            self.master[p + "ff.down_weights"].copy_(
                get(p + "ff.down_weights")[r * Il:(r + 1) * Il])
            for mine, theirs in (("norm1", n1), ("norm2", n2)):
                self.master[p + mine + "_scale"].copy_(get(p + theirs + "_scale"))
                if not self.rms:
                    self.master[p + mine + "_bias"].copy_(get(p + theirs + "_bias"))
        self.master["output_proj"].copy_(get("output_proj")[:, r * Vl:(r + 1) * Vl])
        self.master["final_norm_scale"].copy_(get(fn + "_scale"))
        if not self.rms:
            self.master["final_norm_bias"].copy_(get(fn + "_bias"))
        self.p16.copy_(self.p32)

    def gather_full(self) -> Dict[str, torch.Tensor]:
        """The unsharded fp32 tensors under the names of :class:`DecoderLM` (``attn.qkv_weights``
        fused, ``ff.gate_up_weights`` for SwiGLU), assembled from all ranks' shards; every rank
        gets the full set.  The inverse of :meth:`load_from_full`."""
        cfg, n = self.cfg, self.n
        H, Hl, Il = cfg.hidden_dim, self.Hl, self.Il
        group = self.tp.group

        def gather(t: torch.Tensor):
            if n == 1:
                return [t]
            parts = [torch.empty_like(t) for _ in range(n)]
            dist.all_gather(parts, t.contiguous(), group=group)
            return parts

        from ..models.decoder import ParamLayout
        n1, n2, fn = ParamLayout(cfg).norm_names
        out: Dict[str, torch.Tensor] = {}
        emb = torch.zeros((cfg.vocab_padded, H), dtype=torch.float32, device=self.device)
        emb[:cfg.vocab_size] = self.master["token_embed"]
        out["token_embed"] = emb
        for l in range(cfg.num_layers):
            p = f"layers.{l}."
            qkv = gather(self.master[p + "attn.qkv_weights"])
            Kl = self.Kl
            out[p + "attn.qkv_weights"] = torch.cat(
                [torch.cat([s[:, lo:hi] for s in qkv], 1)
                 for lo, hi in ((0, Hl), (Hl, Hl + Kl), (Hl + Kl, Hl + 2 * Kl))], 1)
            out[p + "attn.o_weights"] = torch.cat(gather(self.master[p + "attn.o_weights"]), 0)
            up = gather(self.master[p + "ff.up_weights"])
            if self.swiglu:
                out[p + "ff.gate_up_weights"] = torch.cat(
                    [torch.cat([s[:, :Il] for s in up], 1), torch.cat([s[:, Il:] for s in up], 1)], 1)
            else:
                out[p + "ff.up_weights"] = torch.cat(up, 1)
            out[p + "ff.down_weights"] = torch.cat(gather(self.master[p + "ff.down_weights"]), 0)
            for mine, theirs in (("norm1", n1), ("norm2", n2)):
                out[p + theirs + "_scale"] = self.master[p + mine + "_scale"].clone()
                if not self.rms:
                    out[p + theirs + "_bias"] = self.master[p + mine + "_bias"].clone()
        out["output_proj"] = torch.cat(gather(self.master["output_proj"]), 1)
        out[fn + "_scale"] = self.master["final_norm_scale"].clone()
        if not self.rms:
            out[fn + "_bias"] = self.master["final_norm_bias"].clone()
        return out

    def save(self, path: str, fmt: Optional[str] = None) -> None:
        """Write the whole model (``.safetensors`` / ``.gguf`` / ``.rustllm``) from rank 0; the
        file loads into an unsharded model or, through :meth:`load_from_full` or the
        tensor-parallel slicer of the checkpoint module, into any tensor-parallel degree."""
        full = self.gather_full()
        if self.rank == 0:
            from ..checkpoint.formats import save_model

            class _View:
                cfg = self.cfg

                @staticmethod
                def named_parameters():
                    return full.items()
            save_model(_View, path, fmt)
        if self.n > 1:
            dist.barrier(group=self.tp.group)

    def num_parameters_local(self) -> int:
        return sum(math.prod(s) for _, s, _ in self.specs)

    def zero_grad(self) -> None:
        self.g32.zero_()

    def _norm(self, x, prefix):
        return N.norm_fwd(x, self.w[prefix + "_scale"],
                          None if self.rms else self.w[prefix + "_bias"], self.cfg.norm_eps, self.rms)

    def _norm_bwd(self, dy, x, prefix, mean, rstd, dres):
        return N.norm_bwd(dy, x, self.w[prefix + "_scale"], mean, rstd, self.g[prefix + "_scale"],
                          None if self.rms else self.g[prefix + "_bias"], dres, self.rms)

    def _positions(self, S: int):
        if self.cfg.pos != "sinusoidal":
            return None
        if self._pe is None or self._pe.shape[0] < S:
            self._pe = E.sinusoid_table(max(S, self.cfg.max_seq_len), self.cfg.hidden_dim, self.device)
        return self._pe

    # ------------------------------------------------------------------ forward
    def _rope(self, qkv: torch.Tensor, S: int, inverse: bool = False, pos_offset: int = 0,
              pos_dev: Optional[torch.Tensor] = None) -> None:
        """Rotary embedding of this rank's query and K/V heads (adjacent in the fused buffer);
        Llama-3.1 style scaled frequencies go through the explicit frequency table."""
        cfg, heads = self.cfg, self.nh_l + self.kvh_l
        if cfg.rope_llama3 is not None:
            if getattr(self, "_inv_freq", None) is None:
                f, lo, hi, orig = cfg.rope_llama3
                self._inv_freq = E.llama3_inv_freq(cfg.head_dim, cfg.rope_theta, f, lo, hi,
                                                   int(orig)).to(self.device)
            E.rope_freq_(qkv, heads, cfg.head_dim, S, self._inv_freq, pos_offset=pos_offset,
                         inverse=inverse, pos_dev=pos_dev)
        else:
            E.rope_(qkv, heads, cfg.head_dim, S, pos_offset=pos_offset, theta=cfg.rope_theta,
                    inverse=inverse, pos_dev=pos_dev)

    def _split_qkv(self, qkv: torch.Tensor, expand: bool = True):
        """``(q, k, v)`` of this rank's heads; under grouped-query attention ``expand=True``
        repeats the rank's K/V heads for the query heads of their groups (``[T, Hl]`` each: the
        backward attention kernel is multi-head), ``expand=False`` leaves K/V ``[T, Kl]`` (the
        forward, decode and cache-write kernels index them by query head // group)."""
        Hl, Kl = self.Hl, self.Kl
        q, k, v = qkv[:, :Hl], qkv[:, Hl:Hl + Kl], qkv[:, Hl + Kl:]
        if self.gqa and expand:
            T, dh, g_ = qkv.shape[0], self.cfg.head_dim, self.nh_l // self.kvh_l
            k, v = (t.reshape(T, self.kvh_l, 1, dh).expand(T, self.kvh_l, g_, dh).reshape(T, Hl)
                    for t in (k, v))
        return q, k, v

    def _layer_fwd(self, l: int, x: torch.Tensor, B: int, S: int):
        """One block on this rank's ``[T/tp, H]`` rows; returns the block output and the tensors
        its backward needs."""
        cfg, tp = self.cfg, self.tp
        T = B * S
        H, dh, nh, Hl = cfg.hidden_dim, cfg.head_dim, self.nh_l, self.Hl
        p = f"layers.{l}."
        n1, mean1, rstd1 = self._norm(x, p + "norm1")
        tp.own_rows("ag_attn", T, H).copy_(n1)
        qkv, n1_full = tp.ag_gemm("ag_attn", self.w[p + "attn.qkv_weights"])
        n1_full = n1_full.clone()
        if cfg.pos == "rope":
            self._rope(qkv, S)
        q, k, v = self._split_qkv(qkv)
        attn, lse = A.attention_fwd(q, k, v, B, S, nh, dh, causal=True)
        x_mid = tp.gemm_rs("rs_attn", attn, self.w[p + "attn.o_weights"], resid=x)
        n2, mean2, rstd2 = self._norm(x_mid, p + "norm2")
        tp.own_rows("ag_mlp", T, H).copy_(n2)
        u, n2_full = tp.ag_gemm("ag_mlp", self.w[p + "ff.up_weights"])
        n2_full = n2_full.clone()
        act = E.swiglu_fwd(u) if self.swiglu else E.gelu_fwd(u)
        x_out = tp.gemm_rs("rs_mlp", act, self.w[p + "ff.down_weights"], resid=x_mid)
        return x_out, dict(x=x, mean1=mean1, rstd1=rstd1, n1_full=n1_full, qkv=qkv, attn=attn,
                           lse=lse, x_mid=x_mid, mean2=mean2, rstd2=rstd2, n2_full=n2_full, u=u,
                           act=act)

    def forward_loss(self, ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """``ids``, ``targets``: the SAME ``[B, S]`` batch on every rank of the group.  Returns the
        mean loss (identical on all ranks) and keeps what :meth:`backward` needs."""
        cfg, tp = self.cfg, self.tp
        B, S = ids.shape
        T = B * S
        n, r = self.n, self.rank
        if T % n:
            raise ProcessingError.invalid_input(f"B*S = {T} must be divisible by tp = {n}")
        Ts = T // n
        if Ts % S and S % Ts:
            raise ProcessingError.invalid_input("tokens per rank must divide or be a multiple of S")
        H, dh, nh = cfg.hidden_dim, cfg.head_dim, self.nh_l
        Hl = self.Hl
        my_ids = ids.reshape(-1)[r * Ts:(r + 1) * Ts].contiguous()
        pos_off = (r * Ts) % S if Ts < S else 0
        x = E.embed_fwd(my_ids, self.w["token_embed"], self._positions(S), S, pos_offset=pos_off)
        sv: dict = {"ids": my_ids, "B": B, "S": S, "T": T, "Ts": Ts, "layers": []}
        for l in range(cfg.num_layers):
            x_out, kept = self._layer_fwd(l, x, B, S)
            sv["layers"].append(dict(x=x) if self.recompute else kept)
            x = x_out
        xf, meanf, rstdf = self._norm(x, "final_norm")
        tp.own_rows("ag_head", T, H).copy_(xf)
        logits, xf_full = tp.ag_gemm("ag_head", self.w["output_proj"])
        sv.update(x_last=x, meanf=meanf, rstdf=rstdf, xf_full=xf_full.clone())
        # vocabulary-parallel cross entropy: exchange (max, sum-exp, target logit) per token
        V, Vl = cfg.vocab_size, self.Vl
        v0 = r * Vl
        width = max(0, min(Vl, V - v0))          # real (unpadded) columns of this shard
        tg = targets.reshape(-1)
        stats = E.cross_entropy_stats(logits[:, :max(width, 1)] if width else logits[:, :1], tg, v0)
        if width == 0:
            stats[:, 0] = float("-inf"); stats[:, 1] = 0; stats[:, 2] = 0
        allst = [torch.empty_like(stats) for _ in range(n)]
        if n > 1:
            dist.all_gather(allst, stats, group=tp.group)
        else:
            allst = [stats]
        st = torch.stack(allst)                                    # [n, T, 3]
        gm = st[:, :, 0].max(0).values
        gs = (st[:, :, 1] * torch.exp(st[:, :, 0] - gm)).sum(0)
        lse_tok = gm + torch.log(gs)
        tl = st[:, :, 2].sum(0)
        valid = (tg >= 0).float()
        loss = ((lse_tok - tl) * valid).sum() / T
        if width:
            E.cross_entropy_bwd_from_lse(logits[:, :width], tg, lse_tok.contiguous(), v0, 1.0 / T)
        if width < Vl:
            logits[:, width:] = 0
        sv["dlogits"] = logits
        self._saved = sv
        return loss.reshape(1)

    # ------------------------------------------------------------------ backward
    def backward(self) -> None:
        """Gradients of the local shards (fp32, accumulated); replicated parameters (norms,
        embedding) are summed over the group at the end because every rank saw different tokens."""
        sv = self._saved
        if sv is None:
            raise ProcessingError.not_initialized("backward (no forward_loss saved)")
        cfg, tp = self.cfg, self.tp
        B, S, T = sv["B"], sv["S"], sv["T"]
        H, dh, nh, Hl = cfg.hidden_dim, cfg.head_dim, self.nh_l, self.Hl
        dlog = sv["dlogits"]
        G.linear_wgrad(sv["xf_full"], dlog, self.g["output_proj"])
        dxf = tp.gemm_rs("rs_head_b", dlog, self.w["output_proj"], b_mn=False)
        dx = self._norm_bwd(dxf, sv["x_last"], "final_norm", sv["meanf"], sv["rstdf"], None)
        for l in reversed(range(cfg.num_layers)):
            a = sv["layers"][l]
            if "qkv" not in a:          # activation checkpointing
                a = self._layer_fwd(l, a["x"], B, S)[1]
            p = f"layers.{l}."
            # ---- feed-forward
            tp.own_rows("ag_mlp_b", T, H).copy_(dx)
            dact, dx_full = tp.ag_gemm("ag_mlp_b", self.w[p + "ff.down_weights"], b_mn=False)
            G.linear_wgrad(a["act"], dx_full, self.g[p + "ff.down_weights"])
            du = E.swiglu_bwd(a["u"], dact) if self.swiglu else E.gelu_bwd(a["u"], dact)
            G.linear_wgrad(a["n2_full"], du, self.g[p + "ff.up_weights"])
            dn2 = tp.gemm_rs("rs_mlp_b", du, self.w[p + "ff.up_weights"], b_mn=False)
            dx_mid = self._norm_bwd(dn2, a["x_mid"], p + "norm2", a["mean2"], a["rstd2"], dx)
            # ---- attention
            tp.own_rows("ag_attn_b", T, H).copy_(dx_mid)
            dattn, dxm_full = tp.ag_gemm("ag_attn_b", self.w[p + "attn.o_weights"], b_mn=False)
            G.linear_wgrad(a["attn"], dxm_full, self.g[p + "attn.o_weights"])
            qkv = a["qkv"]
            q, k, v = self._split_qkv(qkv)
            dq, dk, dv = A.attention_bwd(dattn, q, k, v, a["attn"], a["lse"], B, S, nh, dh,
                                         causal=True)
            if self.gqa:
                # a K/V head's gradient is the sum over the query heads of its group
                g_, Tn = nh // self.kvh_l, dq.shape[0]
                dk, dv = (t.reshape(Tn, self.kvh_l, g_, dh).float().sum(2).reshape(
                    Tn, self.Kl).to(dq.dtype) for t in (dk, dv))
                dqkv = torch.cat([dq, dk, dv], 1)
            else:
                dqkv = dq._base if dq._base is not None else torch.cat([dq, dk, dv], 1)
            if cfg.pos == "rope":
                self._rope(dqkv, S, inverse=True)
            G.linear_wgrad(a["n1_full"], dqkv, self.g[p + "attn.qkv_weights"])
            dn1 = tp.gemm_rs("rs_attn_b", dqkv, self.w[p + "attn.qkv_weights"], b_mn=False)
            dx = self._norm_bwd(dn1, a["x"], p + "norm1", a["mean1"], a["rstd1"], dx_mid)
        E.embed_bwd(sv["ids"], dx, self.g["token_embed"])
        if self.n > 1:
            # one all-reduce over the vector tail (all replicated) and one over the embedding
            dist.all_reduce(self.g32[self.decay_end:], group=tp.group)
            dist.all_reduce(self.g["token_embed"], group=tp.group)
        self._saved = None


class TPTrainer:
    """Training step of a tensor-parallel model: every rank applies AdamW to its own shards (the
    replicated tensors receive identical summed gradients, so they stay identical)."""

    def __init__(self, model: TPDecoderLM, opt_cfg=None, dp_group=None, schedule=None) -> None:
        """``dp_group``: ranks that hold the SAME shards in other tensor-parallel groups (data
        parallelism across replicas of the tensor-parallel model); their gradients are averaged
        with one all-reduce of the flat local gradient buffer before the optimizer step."""
        from ..optim.adamw import AdamW, AdamWConfig
        self.model = model
        self.opt = AdamW(opt_cfg or AdamWConfig(), 0, model.n_flat, model.decay_end, model.device)
        self.step_index = 0
        self.schedule = schedule          # object with at(step) -> learning rate
        self.dp_group = dp_group
        self.dp_degree = dist.get_world_size(dp_group) if dp_group is not None else 1
        if model.n > 1:
            # global gradient norm: replicated tensors (embedding, norms) have the same gradient
            # on every rank of the group, the sharded matrices one slice each
            def norm_hook(g32, sumsq):
                rep = torch.zeros_like(sumsq)
                for name in model.replicated:
                    o, shape = model.offsets[name]
                    E.sumsq_into(g32[o:o + math.prod(shape)], rep)
                shards = sumsq - rep
                dist.all_reduce(shards, group=model.tp.group)
                sumsq.copy_(shards + rep)
            self.opt.norm_hook = norm_hook
        if self.dp_degree > 1:      # replicas start from the same weights
            dist.broadcast(model.p32, src=dist.get_global_rank(dp_group, 0), group=dp_group)
            model.p16.copy_(model.p32)

    def train_step(self, ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        m = self.model
        if self.schedule is not None:
            self.opt.set_learning_rate(self.schedule.at(self.step_index))
        m.zero_grad()
        loss = m.forward_loss(ids, targets)
        m.backward()
        if self.dp_degree > 1:
            dist.all_reduce(m.g32, group=self.dp_group)
        self.opt.step(m.p32, m.g32, m.p16, 1.0 / self.dp_degree)
        self.step_index += 1
        return loss

    # ---- training checkpoints: one file per rank (its shards of the weights and moments)
    def save_checkpoint(self, directory: str) -> None:
        """Every rank writes ``tp<rank>.safetensors`` (fp32 master weights and Adam moments of
        its shards); rank 0 adds ``manifest.json``.  Resuming needs the same tensor-parallel
        degree; to change it, :meth:`TPDecoderLM.save` the weights and load them elsewhere."""
        import json
        import os

        from ..checkpoint.formats import save_safetensors
        m = self.model
        os.makedirs(directory, exist_ok=True)
        if m.n > 1:
            dist.barrier(group=m.tp.group)
        save_safetensors(os.path.join(directory, f"tp{m.rank}.safetensors"),
                         {"p32": m.p32, "m": self.opt.m, "v": self.opt.v},
                         {"rank": str(m.rank), "tp": str(m.n)})
        if m.n > 1:
            dist.barrier(group=m.tp.group)
        if m.rank == 0:
            with open(os.path.join(directory, "manifest.json"), "w") as f:
                json.dump({"kind": "tensor-parallel", "tp": m.n, "n_flat": m.n_flat,
                           "opt_step": self.opt.step_count, "train_step": self.step_index,
                           "config": m.cfg.to_dict()}, f)
        if m.n > 1:
            dist.barrier(group=m.tp.group)

    def load_checkpoint(self, directory: str) -> dict:
        import json
        import os

        from ..checkpoint.formats import load_safetensors
        m = self.model
        with open(os.path.join(directory, "manifest.json")) as f:
            man = json.load(f)
        if man.get("kind") != "tensor-parallel" or int(man["tp"]) != m.n \
                or int(man["n_flat"]) != m.n_flat:
            raise ProcessingError.invalid_input(
                f"checkpoint was written at tensor-parallel degree {man.get('tp')} "
                f"({man.get('n_flat')} local elements); this run has degree {m.n} "
                f"({m.n_flat})")
        t, _ = load_safetensors(os.path.join(directory, f"tp{m.rank}.safetensors"))
        m.p32.copy_(t["p32"].to(m.device))
        m.p16.copy_(m.p32)
        self.opt.m.copy_(t["m"].to(m.device))
        self.opt.v.copy_(t["v"].to(m.device))
        self.opt.step_count = int(man["opt_step"])
        self.step_index = int(man["train_step"])
        return man
