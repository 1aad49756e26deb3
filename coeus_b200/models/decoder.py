"""Decoder-only transformer with an explicit forward and backward pass over the hand-written
kernels of :mod:`coeus_b200.ops`.

The math is the reference's forward pass (plugins/model-transformer/src/lib.rs:791-919): token
embedding plus sinusoidal positions, ``num_layers`` pre-norm blocks of causal multi-head
attention and a GELU feed-forward network with residual connections, a final norm and an output
projection ``[H, V]`` without bias.  Weights are stored ``[in, out]`` row-major like the
reference's; Q, K and V are kept as one fused ``[H, 3H]`` matrix so the three projections are one
GEMM.  Normalisation is per token (the reference normalises over the whole ``[S*H]`` buffer,
which equals this at ``S == 1``).  ``DecoderConfig`` additionally selects RMSNorm, rotary
positions and a SwiGLU feed-forward for the larger configurations.

Training state lives in three flat buffers (fp32 master weights, bf16 working copy, fp32
gradients) so that the optimizer, gradient reduction and checkpointing see one contiguous range;
matrices (weight-decayed) come first, vectors (biases, norm scales) after them.  No autograd
graph is built: ``forward_loss`` keeps the activations the hand-written ``backward`` needs.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from ..foundation.error import ProcessingError
from ..ops import attention as A
from ..ops import elementwise as E
from ..ops import gemm as G
from ..ops import norm as N
from .config import DecoderConfig


@dataclass
class ParamSpec:
    name: str
    shape: Tuple[int, ...]
    decay: bool
    kind: str  # "weight" | "bias" | "scale" | "embed"
    offset: int = 0
    expert: bool = False  # rows of dimension 0 are experts, sharded over the expert-parallel group

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


class ParamLayout:
    """Ordered parameter list of a :class:`DecoderConfig` and its placement in the flat buffers.

    Tensor names follow the reference's field names (``token_embed``, ``layers.{l}.ln1_scale``,
    ``layers.{l}.attn.*``, ``layers.{l}.ff.*``, ``final_ln_*``, ``output_proj``) with the fused
    ``attn.qkv_weights`` standing for ``q_weights | k_weights | v_weights``.
    """

    ALIGN = 64  # elements; every tensor starts on a 256-byte (fp32) / 128-byte (bf16) boundary

    def __init__(self, cfg: DecoderConfig, tp: int = 1, ep: int = 1,
                 layers: Optional[Tuple[int, int]] = None, embed: bool = True,
                 head: bool = True) -> None:
        """``layers=(lo, hi)``, ``embed`` and ``head`` restrict the list to one pipeline stage:
        blocks ``lo..hi-1`` (named by their index in the whole model), with or without the
        embedding, and with or without the final norm and LM head."""
        if tp != 1:
            raise ProcessingError.unsupported(
                "a tensor-parallel ParamLayout",
                "tensor-parallel shards are laid out by parallel.tp_model.TPDecoderLM")
        self.cfg = cfg
        self.ep = ep
        self.layer_ids = list(range(*(layers if layers is not None else (0, cfg.num_layers))))
        self.has_embed, self.has_head = embed, head
        if cfg.tie_embeddings and not (embed and head):
            raise ProcessingError.unsupported("tied embeddings across pipeline stages",
                                              "embedding and head would live on different ranks")
        H, I, V, L = cfg.hidden_dim, cfg.intermediate_dim, cfg.vocab_size, cfg.num_layers
        Vp = cfg.vocab_padded
        ln = cfg.norm == "layernorm"
        s1, s2 = ("ln1", "ln2") if ln else ("norm1", "norm2")
        specs: List[ParamSpec] = []
        if embed:
            specs.append(ParamSpec("token_embed", (Vp if cfg.tie_embeddings else V, H), True, "embed"))
            if cfg.pos == "learned":     # trained absolute positions (GPT-2 style)
                specs.append(ParamSpec("pos_embed", (cfg.max_seq_len, H), True, "embed"))
        for l in self.layer_ids:
            p = f"layers.{l}."
            specs.append(ParamSpec(p + "attn.qkv_weights", (H, cfg.qkv_dim), True, "weight"))
            specs.append(ParamSpec(p + "attn.o_weights", (H, H), True, "weight"))
            if cfg.num_experts:
                E_ = cfg.num_experts
                El = E_ // ep   # experts owned by one rank of the expert-parallel group
                specs.append(ParamSpec(p + "moe.router_weights", (H, E_), True, "weight"))
                specs.append(ParamSpec(p + "moe.experts.gate_up_weights", (El, H, 2 * I), True,
                                       "weight", expert=True))
                specs.append(ParamSpec(p + "moe.experts.down_weights", (El, I, H), True,
                                       "weight", expert=True))
            elif cfg.activation == "swiglu":
                specs.append(ParamSpec(p + "ff.gate_up_weights", (H, 2 * I), True, "weight"))
                specs.append(ParamSpec(p + "ff.down_weights", (I, H), True, "weight"))
            else:
                specs.append(ParamSpec(p + "ff.up_weights", (H, I), True, "weight"))
                specs.append(ParamSpec(p + "ff.down_weights", (I, H), True, "weight"))
        if head and not cfg.tie_embeddings:
            specs.append(ParamSpec("output_proj", (H, Vp), True, "weight"))
        vec: List[ParamSpec] = []
        for l in self.layer_ids:
            p = f"layers.{l}."
            vec.append(ParamSpec(p + s1 + "_scale", (H,), False, "scale"))
            if ln:
                vec.append(ParamSpec(p + s1 + "_bias", (H,), False, "bias"))
            vec.append(ParamSpec(p + s2 + "_scale", (H,), False, "scale"))
            if ln:
                vec.append(ParamSpec(p + s2 + "_bias", (H,), False, "bias"))
            if cfg.use_bias:
                vec.append(ParamSpec(p + "attn.qkv_bias", (cfg.qkv_dim,), False, "bias"))
                vec.append(ParamSpec(p + "attn.o_bias", (H,), False, "bias"))
                if not cfg.num_experts and cfg.activation == "gelu":
                    vec.append(ParamSpec(p + "ff.up_bias", (I,), False, "bias"))
                    vec.append(ParamSpec(p + "ff.down_bias", (H,), False, "bias"))
        fn = "final_ln" if ln else "final_norm"
        if head:
            vec.append(ParamSpec(fn + "_scale", (H,), False, "scale"))
            if ln:
                vec.append(ParamSpec(fn + "_bias", (H,), False, "bias"))
        off = 0
        for s in specs + vec:
            s.offset = off
            off += (s.numel + self.ALIGN - 1) // self.ALIGN * self.ALIGN
            if s is specs[-1]:
                self.decay_end = off
        self.specs: List[ParamSpec] = specs + vec
        self.by_name: Dict[str, ParamSpec] = {s.name: s for s in self.specs}
        self.total = off
        self.norm_names = (s1, s2, fn)

    def num_parameters(self) -> int:
        return sum(s.numel for s in self.specs)

    def padded_total(self, multiple: int) -> int:
        return (self.total + multiple - 1) // multiple * multiple


class DecoderLM:
    """The decoder-only language model on one GPU (or on CPU through the ops' oracle path)."""

    def __init__(self, cfg: DecoderConfig, device="cuda", init: str = "normal", seed: int = 0,
                 pad_multiple: int = 8 * 1024, training: bool = True,
                 dtype: torch.dtype = torch.bfloat16, epx=None,
                 layers: Optional[Tuple[int, int]] = None, embed: bool = True,
                 head: bool = True, cp=None, recompute: bool = False,
                 lm_head_chunks: Optional[int] = None) -> None:
        """``lm_head_chunks = n > 1`` (default: ``COEUS_LM_HEAD_CHUNKS``, else 1) computes the LM
        head and the cross-entropy in ``n`` slices of the vocabulary, so that the ``[tokens,
        vocabulary]`` logits are never held at once: per slice the logits go through the
        (max, sum-exp, target-logit) kernel of the vocabulary-parallel loss; the backward pass
        recomputes a slice's logits, turns them into their gradient in place and feeds the head's
        weight- and data-gradient GEMMs from it.  One more LM-head product per step for
        ``1/n`` of the logits memory (1 GB at the benchmark's 16384 x 32000, 4 GB at a 128k
        vocabulary).
        ``recompute=True`` keeps only each block's input for the backward pass and runs the
        block's forward again there (activation checkpointing: about one third more compute for
        a per-layer activation footprint of one ``[T, H]`` tensor instead of roughly
        ``[T, 14 H]``).
        ``cp`` is a :class:`coeus_b200.parallel.cp.ContextParallel` (token ids then come as this
        rank's two zig-zag chunks ``[2, B, Sc]`` and attention runs as ring attention over the
        group) or a :class:`coeus_b200.parallel.ulysses.UlyssesParallel` (ids ``[1, B, S/sp]``,
        all-to-all between sequence and head sharding around attention); ``cp.shard(ids)`` makes
        the local ids.
        ``dtype`` is the working precision of weights and activations: bf16 on the GPU (the
        kernels accept nothing else); fp32 is allowed on CPU, where the ops run their oracle.
        ``epx`` is the :class:`coeus_b200.parallel.ep.ExpertParallel` state of a mixture-of-experts
        configuration (``None``: all experts on this rank)."""
        cfg.validate()
        self.cfg = cfg
        self.device = torch.device(device)
        self.cp = cp
        self.recompute = bool(recompute)
        if lm_head_chunks is None:
            lm_head_chunks = int(os.environ.get("COEUS_LM_HEAD_CHUNKS", "1"))
        self.lm_head_chunks = max(1, int(lm_head_chunks))
        self.gqa = cfg.kv_heads != cfg.num_heads
        if self.gqa and cp is not None:
            raise ProcessingError.unsupported(
                "grouped-query attention with context / Ulysses parallelism",
                "the ring and all-to-all paths exchange one K/V head per query head")
        # dropout (training passes only): masks are a function of (seed, step, call, rank, layer,
        # site), nothing is stored; see _drop()
        self.train_mode = True
        self.dropout_seed, self.dropout_step, self.dropout_rank = seed, 0, 0
        self._drop_call, self._drop_active = 0, False
        if cfg.num_experts or cp is not None or layers is not None:
            cfg.require_no_dropout("expert / context / pipeline parallelism")
        self.epx = None
        self.moe: List = []
        if cfg.num_experts:
            from ..parallel.ep import ExpertParallel
            self.epx = epx if epx is not None else ExpertParallel(None, self.device)
            if cfg.num_experts % self.epx.ep:
                raise ProcessingError.invalid_input(
                    "num_experts must be divisible by the expert-parallel degree")
        self.layout = ParamLayout(cfg, ep=self.epx.ep if self.epx is not None else 1,
                                  layers=layers, embed=embed, head=head)
        self.layer_ids = self.layout.layer_ids
        n = self.layout.padded_total(pad_multiple)
        self.n_flat = n
        self.p32 = torch.zeros(n, dtype=torch.float32, device=self.device)
        if self.device.type == "cuda" and cfg.head_dim not in (64, 128):
            raise ProcessingError.unsupported(
                f"head dimension {cfg.head_dim} on CUDA", "the attention kernels cover 64 and 128")
        if self.device.type == "cuda" and dtype != torch.bfloat16:
            raise ProcessingError.unsupported(f"working dtype {dtype} on CUDA", "kernels are bf16")
        self.p16 = torch.zeros(n, dtype=dtype, device=self.device)
        self.g32 = torch.zeros(n, dtype=torch.float32, device=self.device) if training else None
        self.training = training
        self.w: Dict[str, torch.Tensor] = {}
        self.g: Dict[str, torch.Tensor] = {}
        self.master: Dict[str, torch.Tensor] = {}
        self._bind_views()
        self._ws: Dict[str, torch.Tensor] = {}
        self._ws_tag = ""
        self._pe: Optional[torch.Tensor] = None
        self._saved: Optional[dict] = None
        self.max_ctas = 0
        if cfg.num_experts:
            from ..parallel.ep import MoEFFN
            self.moe = [MoEFFN(cfg.hidden_dim, cfg.intermediate_dim, cfg.num_experts, cfg.top_k,
                               cfg.capacity_factor, self.epx, aux_coef=cfg.aux_loss_coef,
                               dtype=dtype, allocate=False) for _ in self.layer_ids]
            self._bind_moe()
        self.init_parameters(init, seed)

    # ------------------------------------------------------------------ parameters
    def _bind_views(self) -> None:
        for s in self.layout.specs:
            sl = slice(s.offset, s.offset + s.numel)
            self.w[s.name] = self.p16[sl].view(s.shape)
            self.master[s.name] = self.p32[sl].view(s.shape)
            if self.g32 is not None:
                self.g[s.name] = self.g32[sl].view(s.shape)
        self._bind_moe()

    def _bind_moe(self) -> None:
        names = {"router": "moe.router_weights", "gate_up": "moe.experts.gate_up_weights",
                 "down": "moe.experts.down_weights"}
        for l, m in zip(self.layer_ids, self.moe):
            p = f"layers.{l}."
            m.bind({k: self.w[p + n] for k, n in names.items()},
                   {k: self.g[p + n] for k, n in names.items()} if self.g32 is not None else {},
                   {k: self.master[p + n] for k, n in names.items()})

    def rebind(self, p16: Optional[torch.Tensor] = None, g32: Optional[torch.Tensor] = None) -> None:
        """Point the views at externally allocated flat buffers (e.g. symmetric memory shared
        with the other data-parallel ranks); current contents are copied over."""
        if p16 is not None:
            p16[: self.n_flat].copy_(self.p16)
            self.p16 = p16[: self.n_flat]
        if g32 is not None:
            if self.g32 is not None:
                g32[: self.n_flat].copy_(self.g32)
            self.g32 = g32[: self.n_flat]
        self._bind_views()

    def init_parameters(self, init: str = "normal", seed: int = 0) -> None:
        """``normal``: weights N(0, init_std) from the PyTorch generator, scales 1, biases 0;
        ``philox``: the same distribution from the counter-based kernel
        (:func:`coeus_b200.ops.elementwise.normal_init_`).  ``reference``: the
        reference's deterministic ``clamp(sin(i * 0.1234567) * sqrt(2/H), ±0.1)`` for every
        element, norm scales and biases included (plugins/model-transformer/src/lib.rs:604-611);
        ``i`` is the element's index in the reference's flat layout."""
        cfg = self.cfg
        if init == "reference":
            from .layout_ref import reference_offsets
            offs = reference_offsets(cfg)
            for name, (off, shape) in offs.items():
                flat = torch.empty(int(math.prod(shape)), dtype=torch.float32, device=self.device)
                E.sin_init_(flat, cfg.hidden_dim, index_offset=off)
                self._assign_reference_tensor(name, flat.view(shape))
        elif init == "normal":
            import zlib
            gen = torch.Generator(device=self.device)
            for s in self.layout.specs:
                t = self.master[s.name]
                # one stream per tensor name: the values do not depend on which other tensors
                # this rank holds (pipeline stages, expert shards)
                gen.manual_seed(seed * 1000003 + zlib.crc32(s.name.encode()))
                if s.expert and self.layout.ep > 1:
                    # every rank draws all experts and keeps its own, so the values do not
                    # depend on the expert-parallel degree
                    El = s.shape[0]
                    full = torch.empty((El * self.layout.ep,) + tuple(s.shape[1:]),
                                       dtype=torch.float32, device=self.device)
                    full.normal_(0.0, cfg.init_std, generator=gen)
                    t.copy_(full[self.epx.rank * El:(self.epx.rank + 1) * El])
                    del full
                elif s.kind in ("weight", "embed"):
                    t.normal_(0.0, cfg.init_std, generator=gen)
                elif s.kind == "scale":
                    t.fill_(1.0)
                else:
                    t.zero_()
        elif init == "philox":
            # counter-based N(0, init_std) drawn by the framework's own kernel: one key per tensor
            # name, the element index as counter, so every shard (expert slice, pipeline stage,
            # CPU or GPU) holds the values of the whole tensor at its place
            import zlib
            for s in self.layout.specs:
                t = self.master[s.name]
                if s.kind in ("weight", "embed"):
                    off = self.epx.rank * t.numel() if (s.expert and self.layout.ep > 1) else 0
                    E.normal_init_(t, (seed << 32) ^ zlib.crc32(s.name.encode()), 0.0,
                                   cfg.init_std, index_offset=off)
                elif s.kind == "scale":
                    t.fill_(1.0)
                else:
                    t.zero_()
        elif init == "zeros":
            self.p32.zero_()
        else:
            raise ProcessingError.invalid_input(f"unknown init '{init}'")
        V = cfg.vocab_size
        if cfg.vocab_padded != V:   # padding columns / rows of the vocabulary stay zero
            if cfg.tie_embeddings:
                self.master["token_embed"][V:].zero_()
            elif "output_proj" in self.master:
                self.master["output_proj"][:, V:].zero_()
        self.sync_working_copy()

    def _assign_reference_tensor(self, name: str, value: torch.Tensor) -> None:
        """Store a tensor given under its reference name (q/k/v separate) into the fused layout."""
        H, Hkv = self.cfg.hidden_dim, self.cfg.kv_dim
        spans = {"q": (0, H), "k": (H, H + Hkv), "v": (H + Hkv, H + 2 * Hkv)}
        for part, (lo, hi) in spans.items():
            if name.endswith(f"attn.{part}_weights"):
                fused = name.replace(f"attn.{part}_weights", "attn.qkv_weights")
                self.master[fused][:, lo:hi] = value
                return
            if name.endswith(f"attn.{part}_bias"):
                fused = name.replace(f"attn.{part}_bias", "attn.qkv_bias")
                self.master[fused][lo:hi] = value
                return
        dst = self.master[name]
        if tuple(dst.shape) != tuple(value.shape):   # vocabulary padding
            dst.zero_()
            dst[tuple(slice(0, n) for n in value.shape)] = value
        else:
            dst.copy_(value)

    def sync_working_copy(self) -> None:
        self.p16.copy_(self.p32)

    def num_parameters(self) -> int:
        return self.layout.num_parameters()

    def named_parameters(self):
        for s in self.layout.specs:
            yield s.name, self.master[s.name]

    # ------------------------------------------------------------------ workspace
    def _buf(self, name: str, shape, dtype=None) -> torch.Tensor:
        key = self._ws_tag + name   # the tag separates micro-batches that are in flight together
        dtype = dtype or self.p16.dtype
        t = self._ws.get(key)
        if t is None or tuple(t.shape) != tuple(shape) or t.dtype != dtype:
            t = torch.empty(shape, dtype=dtype, device=self.device)
            self._ws[key] = t
        return t

    def _positions(self, S: int) -> Optional[torch.Tensor]:
        if self.cfg.pos == "learned":
            # the embedding kernel adds an fp32 table; the working copy is the one every
            # data-parallel rank keeps current
            w = self.w["pos_embed"]
            if S > w.shape[0]:           # the table has one row per trained position, no more
                raise ProcessingError.limit_exceeded("sequence length", w.shape[0], S)
            return w if w.dtype == torch.float32 else w.float()
        if self.cfg.pos != "sinusoidal":
            return None
        if self._pe is None or self._pe.shape[0] < S:
            self._pe = E.sinusoid_table(max(S, self.cfg.max_seq_len), self.cfg.hidden_dim,
                                        self.device)
        return self._pe

    # ------------------------------------------------------------------ forward
    def _norm(self, x, prefix):
        cfg = self.cfg
        rms = cfg.norm == "rmsnorm"
        return N.norm_fwd(x, self.w[prefix + "_scale"], None if rms else self.w[prefix + "_bias"],
                          cfg.norm_eps, rms)

    def rope_inv_freq(self) -> torch.Tensor:
        """Frequency table of a scaled rotary embedding (cached on the model's device)."""
        if getattr(self, "_inv_freq", None) is None:
            f, lo, hi, orig = self.cfg.rope_llama3
            self._inv_freq = E.llama3_inv_freq(self.cfg.head_dim, self.cfg.rope_theta, f, lo, hi,
                                               int(orig)).to(self.device)
        return self._inv_freq

    def _rope(self, qkv: torch.Tensor, B: int, S: int, inverse: bool) -> None:
        """Rotary embedding of the q and k heads (adjacent in the fused buffer); under context
        parallelism each of the two chunks starts at its own position."""
        cfg = self.cfg
        nh, dh = cfg.num_heads, cfg.head_dim
        if cfg.rope_llama3 is not None:
            if self.cp is not None:
                raise ProcessingError.unsupported("scaled rotary embeddings under context "
                                                  "parallelism", "plain RoPE only there")
            E.rope_freq_(qkv, nh + cfg.kv_heads, dh, S, self.rope_inv_freq(), inverse=inverse)
            return
        if self.cp is None:
            # q heads and k heads sit next to each other in the fused buffer
            E.rope_(qkv, nh + cfg.kv_heads, dh, S, theta=cfg.rope_theta, inverse=inverse)
            return
        Tc = B * S
        for c, off in enumerate(self.cp.position_offsets(S)):
            E.rope_(qkv[c * Tc:(c + 1) * Tc], 2 * nh, dh, S, pos_offset=off, theta=cfg.rope_theta,
                    inverse=inverse)

    def train(self, mode: bool = True) -> "DecoderLM":
        """Training mode applies dropout in :meth:`forward_loss`; evaluation mode never does."""
        self.train_mode = bool(mode)
        return self

    def _drop(self, rate: float, l: int, site: int):
        """``(threshold, key)`` of one dropout site of the current training pass, or ``None``
        when dropout does not apply (rate 0, evaluation mode, inference entry points)."""
        if not self._drop_active or not rate:
            return None
        thr = E.dropout_threshold(rate)
        if thr == 0:
            return None
        return thr, E.dropout_key(self.dropout_seed, self.dropout_step, self._drop_call,
                                  self.dropout_rank, l, site)

    def _expand_kv(self, t: torch.Tensor) -> torch.Tensor:
        """``[T, kv_heads * dh] -> [T, heads * dh]``: every K/V head repeated for the query heads
        of its group (query head ``h`` reads K/V head ``h // group``).  The forward kernel reads
        the narrow K/V directly; the backward kernel is multi-head and runs on the expanded
        copies, after which the gradients of a group are summed."""
        cfg = self.cfg
        T, g = t.shape[0], cfg.num_heads // cfg.kv_heads
        return t.reshape(T, cfg.kv_heads, 1, cfg.head_dim).expand(
            T, cfg.kv_heads, g, cfg.head_dim).reshape(T, cfg.hidden_dim)

    def _block_fwd(self, l: int, x: torch.Tensor, B: int, S: int, save: Optional[dict]):
        cfg = self.cfg
        H, nh, dh = cfg.hidden_dim, cfg.num_heads, cfg.head_dim
        p = f"layers.{l}."
        n1n, n2n, _ = self.layout.norm_names
        bias = (lambda n: self.w[p + n]) if cfg.use_bias else (lambda n: None)
        T = x.shape[0]
        mc = self.max_ctas
        n1, mean1, rstd1 = self._norm(x, p + n1n)
        qkv = G.linear_fwd(n1, self.w[p + "attn.qkv_weights"], bias("attn.qkv_bias"),
                           out=self._buf(f"qkv{l}" if save is not None and not self.recompute else "qkv",
                                         (T, cfg.qkv_dim)),
                           max_ctas=mc)
        if cfg.pos == "rope":
            self._rope(qkv, B, S, False)
        if self.cp is not None:
            attn, lse = self.cp.attention_fwd(qkv, B, S, nh, dh)
        else:
            Hkv = cfg.kv_dim
            q, k, v = qkv[:, :H], qkv[:, H:H + Hkv], qkv[:, H + Hkv:]
            # dropout on the probabilities happens inside the flash kernel (the materialised path
            # where it cannot: see ops/attention.py); grouped-query attention: the forward kernel
            # indexes K/V by head // group itself
            da = self._drop(cfg.attention_dropout, l, 2)
            attn, lse = A.attention_fwd(q, k, v, B, S, nh, dh, causal=True, dropout=da)
        d0, d1 = self._drop(cfg.dropout, l, 0), self._drop(cfg.dropout, l, 1)
        x_mid = G.linear_fwd(attn, self.w[p + "attn.o_weights"], bias("attn.o_bias"), resid=x,
                             max_ctas=mc, dropout=d0)
        n2, mean2, rstd2 = self._norm(x_mid, p + n2n)
        if self.moe:
            u = act = None
            x_out = self.moe[l - self.layer_ids[0]].forward(n2, x_mid, save=save is not None)
        elif cfg.activation == "swiglu":
            gu = G.linear_fwd(n2, self.w[p + "ff.gate_up_weights"], None, max_ctas=mc)
            act = E.swiglu_fwd(gu)
            u = gu
            x_out = G.linear_fwd(act, self.w[p + "ff.down_weights"], None, resid=x_mid, max_ctas=mc,
                                 dropout=d1)
        else:
            u = torch.empty((T, cfg.intermediate_dim), dtype=self.p16.dtype, device=x.device) \
                if save is not None else None
            act = G.linear_fwd(n2, self.w[p + "ff.up_weights"], bias("ff.up_bias"), epi="gelu",
                               aux_out=u, max_ctas=mc)
            x_out = G.linear_fwd(act, self.w[p + "ff.down_weights"], bias("ff.down_bias"),
                                 resid=x_mid, max_ctas=mc, dropout=d1)
        if save is not None:
            save[l] = dict(x=x, n1=n1, mean1=mean1, rstd1=rstd1, qkv=qkv, attn=attn, lse=lse,
                           x_mid=x_mid, n2=n2, mean2=mean2, rstd2=rstd2, u=u, act=act,
                           drop=(d0, d1, self._drop(cfg.attention_dropout, l, 2)
                                 if self.cp is None else None))
        return x_out

    def _check_ids(self, ids: torch.Tensor) -> Tuple[int, int]:
        if self.cp is not None:
            nc = self.cp.n_chunks
            if ids.dim() != 3 or ids.shape[0] != nc:
                raise ProcessingError.invalid_input(
                    f"sequence parallelism expects ids [{nc}, B, S_local] (use its shard())")
            B, S = ids.shape[1], ids.shape[2]
            if S * nc * self.cp.cp > self.cfg.max_seq_len:
                raise ProcessingError.invalid_input(
                    f"Sequence length {S * nc * self.cp.cp} out of range [1, {self.cfg.max_seq_len}]")
            return B, S
        if ids.dim() == 1:
            ids = ids[None]
        B, S = ids.shape
        if S < 1 or S > self.cfg.max_seq_len:
            raise ProcessingError.invalid_input(
                f"Sequence length {S} out of range [1, {self.cfg.max_seq_len}]")
        return B, S

    def forward_hidden(self, ids: torch.Tensor, save: Optional[dict] = None) -> torch.Tensor:
        """Final-norm output ``[B*S, H]`` for ``ids [B, S]`` (int64)."""
        B, S = self._check_ids(ids)
        x = self.embed(ids, B, S)
        x = self.forward_blocks(x, B, S, save)
        return self.forward_final_norm(x, save)

    def embed(self, ids: torch.Tensor, B: int, S: int) -> torch.Tensor:
        table = self.w["token_embed"]
        if self.cp is None:
            return E.embed_fwd(ids.reshape(-1), table, self._positions(S), S)
        pe = self._positions(S * self.cp.n_chunks * self.cp.cp)
        return torch.cat([E.embed_fwd(ids[c].reshape(-1), table, pe, S, pos_offset=off)
                          for c, off in enumerate(self.cp.position_offsets(S))], 0)

    def forward_blocks(self, x: torch.Tensor, B: int, S: int, save: Optional[dict]) -> torch.Tensor:
        """This model's blocks applied to ``x [B*S, H]``."""
        for l in self.layer_ids:
            if save is not None and self.recompute:
                save[l] = dict(x=x)      # the block runs again in backward_blocks
                x = self._block_fwd(l, x, B, S, None)
            else:
                x = self._block_fwd(l, x, B, S, save)
        return x

    def forward_final_norm(self, x: torch.Tensor, save: Optional[dict]) -> torch.Tensor:
        fn = self.layout.norm_names[2]
        xf, meanf, rstdf = self._norm(x, fn)
        if save is not None:
            save["final"] = dict(x=x, xf=xf, mean=meanf, rstd=rstdf)
        return xf

    def output_weight(self) -> Tuple[torch.Tensor, bool]:
        """``(weight, b_mn)`` of the LM head as the GEMM's B operand."""
        if self.cfg.tie_embeddings:
            return self.w["token_embed"], False   # [V, H] is already [N, K]
        return self.w["output_proj"], True        # [H, V] = [K, N]

    def forward_logits(self, ids: torch.Tensor, last_only: bool = False) -> torch.Tensor:
        """Logits in bf16: ``[B, S, V]``, or ``[B, V]`` of the last position (the reference's
        ``forward`` returns the last position only, lib.rs:913-918)."""
        B, S = self._check_ids(ids)
        self._drop_active = False          # inference entry point: never any dropout
        xf = self.forward_hidden(ids)
        V, Vp = self.cfg.vocab_size, self.cfg.vocab_padded
        if last_only:
            xf = xf.view(B, S, -1)[:, -1, :].contiguous()
        w, b_mn = self.output_weight()
        logits = G.gemm(xf, w, b_mn=b_mn, max_ctas=self.max_ctas)
        return logits.view(B, Vp)[:, :V] if last_only else logits.view(B, S, Vp)[..., :V]

    def forward_loss(self, ids: torch.Tensor, targets: torch.Tensor,
                     grad_scale: Optional[float] = None) -> torch.Tensor:
        """Mean next-token cross-entropy (fp32 scalar tensor) of ``ids [B,S]`` against
        ``targets [B,S]``; keeps what :meth:`backward` needs.  ``grad_scale`` is the factor the
        logit gradients are multiplied with (default ``1 / (B*S)``)."""
        B, S = self._check_ids(ids)
        cfg = self.cfg
        self._drop_active = bool(self.train_mode and self.g32 is not None
                                 and (cfg.dropout or cfg.attention_dropout))
        if self._drop_active:
            self._drop_call += 1           # micro-steps of one optimizer step draw different masks
        save: dict = {"ids": ids.reshape(-1), "B": B, "S": S}
        xf = self.forward_hidden(ids, save)
        return self.loss_from_hidden(xf, targets, save, grad_scale)

    def loss_from_hidden(self, xf: torch.Tensor, targets: torch.Tensor, save: dict,
                         grad_scale: Optional[float] = None) -> torch.Tensor:
        """LM head and cross-entropy on the final-norm output; stores ``save`` for backward."""
        T = xf.shape[0]
        w, b_mn = self.output_weight()
        scale = grad_scale if grad_scale is not None else 1.0 / T
        if self.lm_head_chunks > 1:
            loss_tok = self._chunked_head_loss(xf, targets.reshape(-1), save, scale)
        else:
            logits = G.gemm(xf, w, b_mn=b_mn, out=self._buf("logits", (T, self.cfg.vocab_padded)),
                            max_ctas=self.max_ctas)
            loss_tok = E.cross_entropy_fwd_bwd(logits, targets.reshape(-1), scale,
                                               vocab=self.cfg.vocab_size)
            save["dlogits"] = logits
        save["aux_scale"] = scale * T   # the auxiliary losses follow the scaling of the main loss
        self._saved = save
        loss = torch.zeros(1, dtype=torch.float32, device=self.device)
        E.sum_scaled_into(loss_tok, loss, 1.0 / T)
        self.last_ce = loss
        if self.moe:   # router load-balancing terms (already multiplied by their coefficient)
            loss = loss + torch.stack([m.last_aux for m in self.moe]).sum()
        return loss

    # ---- LM head and loss in slices of the vocabulary (lm_head_chunks > 1)
    def _head_chunks(self) -> List[Tuple[int, int, int]]:
        """``(first column, end column, valid columns)`` of every slice of the padded vocabulary;
        widths are multiples of 256 columns."""
        V, Vp = self.cfg.vocab_size, self.cfg.vocab_padded
        width = -(-Vp // self.lm_head_chunks)
        width = -(-width // 256) * 256
        return [(c0, min(Vp, c0 + width), max(0, min(V, c0 + width) - c0))
                for c0 in range(0, Vp, width)]

    def _head_slice_logits(self, xf: torch.Tensor, c0: int, c1: int) -> torch.Tensor:
        w, b_mn = self.output_weight()
        wc = w[:, c0:c1] if b_mn else w[c0:c1]
        buf = self._buf("logits_slice", (xf.shape[0], self._head_chunks()[0][1]))
        return G.gemm(xf, wc, b_mn=b_mn, out=buf[:, :c1 - c0], max_ctas=self.max_ctas)

    def _chunked_head_loss(self, xf: torch.Tensor, targets: torch.Tensor, save: dict,
                           scale: float) -> torch.Tensor:
        """Per-token loss from per-slice (max, sum-exp, target-logit) statistics."""
        m = s = tl = None
        for c0, c1, valid in self._head_chunks():
            if valid == 0:
                continue
            st = E.cross_entropy_stats(self._head_slice_logits(xf, c0, c1)[:, :valid], targets, c0)
            if m is None:
                m, s, tl = st[:, 0].clone(), st[:, 1].clone(), st[:, 2].clone()
            else:
                mn = torch.maximum(m, st[:, 0])
                s = s * torch.exp(m - mn) + st[:, 1] * torch.exp(st[:, 0] - mn)
                m, tl = mn, tl + st[:, 2]
        lse = m + torch.log(s)
        save["head_chunked"] = {"lse": lse, "targets": targets, "scale": scale}
        return (lse - tl) * (targets >= 0)

    def _chunked_head_backward(self, sv: dict) -> torch.Tensor:
        """Head gradients slice by slice; returns d loss / d (final-norm output) in bf16."""
        hc, xf = sv["head_chunked"], sv["final"]["xf"]
        w, b_mn = self.output_weight()
        mc = self.max_ctas
        dxf = torch.zeros((xf.shape[0], xf.shape[1]), dtype=torch.float32, device=xf.device)
        for c0, c1, valid in self._head_chunks():
            dlog = self._head_slice_logits(xf, c0, c1)
            if valid > 0:
                E.cross_entropy_bwd_from_lse(dlog[:, :valid], hc["targets"], hc["lse"], c0,
                                             hc["scale"])
            if valid < c1 - c0:
                dlog[:, valid:].zero_()      # padding columns of the vocabulary: no gradient
            if self.cfg.tie_embeddings:
                G.gemm(dlog, xf, a_mn=True, b_mn=True, out=self.g["token_embed"][c0:c1],
                       accumulate=True, ksplit=2, max_ctas=mc)
                G.gemm(dlog, w[c0:c1], b_mn=True, out=dxf, accumulate=True, max_ctas=mc)
            else:
                G.linear_wgrad(xf, dlog, self.g["output_proj"][:, c0:c1], max_ctas=mc)
                G.gemm(dlog, w[:, c0:c1], out=dxf, accumulate=True, max_ctas=mc)
        return dxf.to(xf.dtype)

    # ------------------------------------------------------------------ backward
    def zero_grad(self) -> None:
        self.g32.zero_()

    def backward(self, on_layer_done=None) -> None:
        """Accumulate parameter gradients (fp32) for the last :meth:`forward_loss`.
        ``on_layer_done(l)`` is called once the gradients of layer ``l`` are complete (``-1`` for
        the LM head and final norm, ``-2`` after the embedding), which is where the data-parallel
        reduction of a bucket may start."""
        sv = self._saved
        if sv is None:
            raise ProcessingError.not_initialized("backward (no forward_loss saved)")
        dx = self.backward_head(sv)
        if on_layer_done is not None:
            on_layer_done(-1)
        dx = self.backward_blocks(dx, sv, on_layer_done)
        E.embed_bwd(sv["ids"], dx, self.g["token_embed"])
        self.backward_positions(dx, sv)
        if on_layer_done is not None:
            on_layer_done(-2)
        self._saved = None

    def backward_positions(self, dx: torch.Tensor, sv: dict) -> None:
        """Gradient of a learned position table: row ``s`` collects ``dx`` of position ``s`` of
        every sequence (the embedding-gradient kernel with the positions as ids)."""
        if self.cfg.pos != "learned":
            return
        if self.cp is not None:
            raise ProcessingError.unsupported("learned positions under context parallelism",
                                              "use rotary or sinusoidal positions")
        S = sv["S"]
        pos_ids = torch.arange(dx.shape[0], device=dx.device, dtype=torch.int64) % S
        E.embed_bwd(pos_ids, dx, self.g["pos_embed"])

    def backward_head(self, sv: dict) -> torch.Tensor:
        """Gradients of the LM head and final norm; returns d loss / d (last block output)."""
        cfg = self.cfg
        rms = cfg.norm == "rmsnorm"
        fn = self.layout.norm_names[2]
        mc = self.max_ctas
        fin = sv["final"]
        # the result is the gradient of the last block's output: its column sums are the bias
        # gradient of that block's down projection, taken by the same kernel
        cols = None
        if self.layer_ids and self._down_bias_rides_on_norm():
            last = self.layer_ids[-1]
            cols = self.g[f"layers.{last}.ff.down_bias"]
            sv["down_bias_summed"] = last
        if "head_chunked" in sv:
            dxf = self._chunked_head_backward(sv)
            return N.norm_bwd(dxf, fin["x"], self.w[fn + "_scale"], fin["mean"], fin["rstd"],
                              self.g[fn + "_scale"], None if rms else self.g[fn + "_bias"], None,
                              rms, colsum=cols)
        dlog = sv["dlogits"]
        w, b_mn = self.output_weight()
        if cfg.tie_embeddings:
            # d token_embed[V,H] += dlogits^T[V,T] @ xf[T,H]
            G.gemm(dlog, fin["xf"], a_mn=True, b_mn=True, out=self.g["token_embed"],
                   accumulate=True, ksplit=2, max_ctas=mc)
            dxf = G.gemm(dlog, w, b_mn=True, max_ctas=mc)
        else:
            G.linear_wgrad(fin["xf"], dlog, self.g["output_proj"], max_ctas=mc)
            dxf = G.linear_dgrad(dlog, w, max_ctas=mc)
        return N.norm_bwd(dxf, fin["x"], self.w[fn + "_scale"], fin["mean"], fin["rstd"],
                          self.g[fn + "_scale"], None if rms else self.g[fn + "_bias"], None, rms,
                          colsum=cols)

    def _bias_rides_on_norm(self) -> bool:
        """Whether the bias gradients of the projections that write into the residual stream are
        summed by the norm-backward kernel that produces that stream's gradient (not when
        residual dropout scales the gradient between the two)."""
        return bool(self.cfg.use_bias and not (self._drop_active and self.cfg.dropout))

    def _down_bias_rides_on_norm(self) -> bool:
        return bool(self._bias_rides_on_norm() and not self.moe
                    and self.cfg.activation != "swiglu")

    def backward_blocks(self, dx: torch.Tensor, sv: dict, on_layer_done=None) -> torch.Tensor:
        """Backward through this model's blocks; returns d loss / d (first block input)."""
        cfg = self.cfg
        H, nh, dh = cfg.hidden_dim, cfg.num_heads, cfg.head_dim
        B, S = sv["B"], sv["S"]
        rms = cfg.norm == "rmsnorm"
        n1n, n2n, fn = self.layout.norm_names
        mc = self.max_ctas
        ride_o, ride_down = self._bias_rides_on_norm(), self._down_bias_rides_on_norm()
        down_summed = sv.pop("down_bias_summed", None)   # layer whose down bias is already done
        for l in reversed(self.layer_ids):
            a = sv[l]
            if "n1" not in a:            # activation checkpointing: rebuild the block's tensors
                again: dict = {}
                self._block_fwd(l, a["x"], B, S, again)
                a = again[l]
            p = f"layers.{l}."
            d0, d1, da = a.get("drop", (None, None, None))
            # the gradient that enters the down projection is the residual gradient times the
            # (recomputed) dropout mask; dx itself continues along the residual path
            dxd = E.dropout_apply(dx, *d1) if d1 is not None else dx
            if self.moe:
                dn2 = self.moe[l - self.layer_ids[0]].backward(dx, aux_grad_scale=sv["aux_scale"])
            elif cfg.activation == "swiglu":
                G.linear_wgrad(a["act"], dxd, self.g[p + "ff.down_weights"], max_ctas=mc)
                dact = G.linear_dgrad(dxd, self.w[p + "ff.down_weights"], max_ctas=mc)
                du = E.swiglu_bwd(a["u"], dact)
                G.linear_wgrad(a["n2"], du, self.g[p + "ff.gate_up_weights"], max_ctas=mc)
                dn2 = G.linear_dgrad(du, self.w[p + "ff.gate_up_weights"], max_ctas=mc)
            else:
                G.linear_wgrad(a["act"], dxd, self.g[p + "ff.down_weights"], max_ctas=mc)
                # the plain data-gradient GEMM followed by the bandwidth-bound GELU-gradient
                # kernel (0.106 + 0.062 ms at 16384 x 4096) beats the GEMM with the GELU gradient
                # in its epilogue (0.231 ms: the per-row reads of the pre-activation stall it)
                dact = G.linear_dgrad(dxd, self.w[p + "ff.down_weights"], max_ctas=mc)
                # ... which also sums its output's columns: the up projection's bias gradient
                du = E.gelu_bwd(a["u"], dact, self.g[p + "ff.up_bias"] if cfg.use_bias else None)
                G.linear_wgrad(a["n2"], du, self.g[p + "ff.up_weights"], max_ctas=mc)
                if cfg.use_bias and down_summed != l:
                    E.colsum_into(dxd, self.g[p + "ff.down_bias"])
                dn2 = G.linear_dgrad(du, self.w[p + "ff.up_weights"], max_ctas=mc)
            # dx_mid is the gradient of the attention block's output: its column sums are the
            # output projection's bias gradient
            dx_mid = N.norm_bwd(dn2, a["x_mid"], self.w[p + n2n + "_scale"], a["mean2"], a["rstd2"],
                                self.g[p + n2n + "_scale"],
                                None if rms else self.g[p + n2n + "_bias"], dx, rms,
                                colsum=self.g[p + "attn.o_bias"] if ride_o else None)
            dxm = E.dropout_apply(dx_mid, *d0) if d0 is not None else dx_mid
            G.linear_wgrad(a["attn"], dxm, self.g[p + "attn.o_weights"], max_ctas=mc)
            if cfg.use_bias and not ride_o:
                E.colsum_into(dxm, self.g[p + "attn.o_bias"])
            dattn = G.linear_dgrad(dxm, self.w[p + "attn.o_weights"], max_ctas=mc)
            qkv = a["qkv"]
            Hkv = cfg.kv_dim
            q, k, v = qkv[:, :H], qkv[:, H:H + Hkv], qkv[:, H + Hkv:]
            dqkv = self._buf("dqkv", (dattn.shape[0], 3 * H))
            if self.cp is not None:
                self.cp.attention_bwd(dattn, qkv, a["attn"], a["lse"], B, S, nh, dh, dqkv=dqkv)
            elif da is not None and not A.flash_dropout_ok(q, S, dh):
                dqkv = self._buf("dqkv_drop", (dattn.shape[0], cfg.qkv_dim))
                A.attention_dropout_bwd(dattn, q, k, v, a["attn"], a["lse"], B, S, nh, dh, *da,
                                        causal=True, dqkv=dqkv)
            elif self.gqa:
                A.attention_bwd(dattn, q, self._expand_kv(k), self._expand_kv(v), a["attn"],
                                a["lse"], B, S, nh, dh, causal=True, dqkv=dqkv, dropout=da)
                # the gradients of a K/V head are the sum over the query heads of its group
                Tn, g = dqkv.shape[0], nh // cfg.kv_heads
                narrow = self._buf("dqkv_gqa", (Tn, cfg.qkv_dim))
                narrow[:, :H].copy_(dqkv[:, :H])
                for j, lo in ((1, H), (2, H + Hkv)):
                    part = dqkv[:, j * H:(j + 1) * H].reshape(Tn, cfg.kv_heads, g, dh)
                    narrow[:, lo:lo + Hkv].copy_(part.float().sum(2).reshape(Tn, Hkv))
                dqkv = narrow
            else:
                A.attention_bwd(dattn, q, k, v, a["attn"], a["lse"], B, S, nh, dh, causal=True,
                                dqkv=dqkv, dropout=da)
            if cfg.pos == "rope":
                self._rope(dqkv, B, S, True)
            G.linear_wgrad(a["n1"], dqkv, self.g[p + "attn.qkv_weights"], max_ctas=mc)
            if cfg.use_bias:
                E.colsum_into(dqkv, self.g[p + "attn.qkv_bias"])
            dn1 = G.linear_dgrad(dqkv, self.w[p + "attn.qkv_weights"], max_ctas=mc)
            # dx is the gradient of the previous block's output: the column sums are that block's
            # down-projection bias gradient
            cols = None
            if ride_down and l - 1 >= self.layer_ids[0]:
                cols = self.g[f"layers.{l - 1}.ff.down_bias"]
                down_summed = l - 1
            dx = N.norm_bwd(dn1, a["x"], self.w[p + n1n + "_scale"], a["mean1"], a["rstd1"],
                            self.g[p + n1n + "_scale"],
                            None if rms else self.g[p + n1n + "_bias"], dx_mid, rms, colsum=cols)
            if on_layer_done is not None:
                on_layer_done(l)
        return dx
