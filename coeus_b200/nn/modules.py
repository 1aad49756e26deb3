"""``torch.nn.Module`` layers over :mod:`coeus_b200.nn.functional`.  Shapes and parameter names
follow the reference's transformer structs (``MultiHeadAttention`` with q/k/v/o weights,
``FeedForward`` with up/down, ``LayerNorm`` scale/bias; plugins/model-transformer/src/lib.rs:131-383)
with q, k and v fused into one matrix."""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from . import functional as F


def _dtype(device) -> torch.dtype:
    return torch.bfloat16 if torch.device(device).type == "cuda" else torch.float32


class Linear(nn.Module):
    """``y = act(x @ W + b)`` with ``W [in, out]``."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 activation: str = "none", device="cuda", init_std: float = 0.02) -> None:
        super().__init__()
        dt = _dtype(device)
        self.weight = nn.Parameter(torch.empty(in_features, out_features, device=device,
                                               dtype=dt).normal_(0, init_std))
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dt)) if bias else None
        self.activation = activation

    def forward(self, x):
        return F.linear(x, self.weight, self.bias, self.activation)


class LayerNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5, device="cuda") -> None:
        super().__init__()
        dt = _dtype(device)
        self.scale = nn.Parameter(torch.ones(dim, device=device, dtype=dt))
        self.bias = nn.Parameter(torch.zeros(dim, device=device, dtype=dt))
        self.eps = eps

    def forward(self, x):
        return F.layer_norm(x, self.scale, self.bias, self.eps)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, device="cuda") -> None:
        super().__init__()
        self.scale = nn.Parameter(torch.ones(dim, device=device, dtype=_dtype(device)))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x, self.scale, self.eps)


class Embedding(nn.Module):
    def __init__(self, vocab: int, dim: int, device="cuda", init_std: float = 0.02) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.empty(vocab, dim, device=device,
                                               dtype=_dtype(device)).normal_(0, init_std))

    def forward(self, ids, pe: Optional[torch.Tensor] = None):
        return F.embedding(ids, self.weight, pe)


class CausalSelfAttention(nn.Module):
    """Fused QKV projection, optional RoPE, flash attention, output projection."""

    def __init__(self, dim: int, num_heads: int, bias: bool = False, rope: bool = False,
                 rope_theta: float = 10000.0, device="cuda", num_kv_heads: int = 0) -> None:
        """``num_kv_heads`` (0 = ``num_heads``): grouped-query attention, K and V projected to
        that many heads and shared by the query heads of a group."""
        super().__init__()
        self.nh, self.dh = num_heads, dim // num_heads
        self.kvh = num_kv_heads or num_heads
        if num_heads % self.kvh:
            raise ValueError("num_kv_heads must divide num_heads")
        self.rope, self.theta = rope, rope_theta
        self.qkv = Linear(dim, dim + 2 * self.kvh * self.dh, bias, device=device)
        self.o = Linear(dim, dim, bias, device=device)

    def forward(self, x, B: int, S: int):
        qkv = self.qkv(x)
        if self.rope:
            qkv = F.rope(qkv, self.nh + self.kvh, self.dh, S, 0, self.theta)
        if self.kvh != self.nh:
            # the attention kernels are multi-head: K/V heads are repeated for their groups
            # (autograd sums the group's gradients back into the narrow projection)
            T, H, Hkv, g = qkv.shape[0], self.nh * self.dh, self.kvh * self.dh, self.nh // self.kvh
            wide = [t.reshape(T, self.kvh, 1, self.dh).expand(T, self.kvh, g, self.dh)
                    .reshape(T, H) for t in (qkv[:, H:H + Hkv], qkv[:, H + Hkv:])]
            qkv = torch.cat([qkv[:, :H]] + wide, 1)
        return self.o(F.attention(qkv, B, S, self.nh, self.dh, True))


class MLP(nn.Module):
    """``down(gelu(up(x)))`` or, with ``swiglu=True``, ``down(silu(gate) * up)``."""

    def __init__(self, dim: int, inter: int, bias: bool = False, swiglu: bool = False,
                 device="cuda") -> None:
        super().__init__()
        self.swiglu = swiglu
        self.up = Linear(dim, 2 * inter if swiglu else inter, bias and not swiglu,
                         activation="none" if swiglu else "gelu", device=device)
        self.down = Linear(inter, dim, bias and not swiglu, device=device)

    def forward(self, x):
        h = self.up(x)
        return self.down(F.swiglu(h) if self.swiglu else h)


class Block(nn.Module):
    """Pre-norm decoder block (the reference's ``TransformerLayer``, lib.rs:425-500)."""

    def __init__(self, dim: int, num_heads: int, inter: int, rms: bool = False, bias: bool = True,
                 swiglu: bool = False, rope: bool = False, device="cuda",
                 num_kv_heads: int = 0) -> None:
        super().__init__()
        Norm = RMSNorm if rms else LayerNorm
        self.norm1, self.norm2 = Norm(dim, device=device), Norm(dim, device=device)
        self.attn = CausalSelfAttention(dim, num_heads, bias, rope, device=device,
                                        num_kv_heads=num_kv_heads)
        self.mlp = MLP(dim, inter, bias, swiglu, device=device)

    def forward(self, x, B: int, S: int):
        x = x + self.attn(self.norm1(x), B, S)
        return x + self.mlp(self.norm2(x))


class CrossEntropyLoss(nn.Module):
    def forward(self, logits, targets):
        return F.cross_entropy(logits, targets)


class TransformerLM(nn.Module):
    """The decoder-only language model of :class:`coeus_b200.models.config.DecoderConfig` as an
    autograd module over the same kernels (dense feed-forward; the explicit
    :class:`coeus_b200.models.decoder.DecoderLM` is the path the trainers and the parallel
    strategies use and also covers mixtures of experts).  ``forward(ids [B, S])`` returns the
    logits ``[B*S, V]``, or the mean next-token loss when ``targets`` is given."""

    def __init__(self, cfg, device="cuda") -> None:
        super().__init__()
        if cfg.num_experts or cfg.rope_llama3 is not None or cfg.pos == "learned":
            raise ValueError("TransformerLM covers dense models with sinusoidal or plain rotary "
                             "positions; use DecoderLM for experts, scaled rotary embeddings "
                             "and learned positions")
        self.cfg = cfg
        H = cfg.hidden_dim
        rms, swiglu, rope = cfg.norm == "rmsnorm", cfg.activation == "swiglu", cfg.pos == "rope"
        self.embed = Embedding(cfg.vocab_size, H, device=device, init_std=cfg.init_std)
        self.blocks = nn.ModuleList([
            Block(H, cfg.num_heads, cfg.intermediate_dim, rms=rms, bias=cfg.use_bias,
                  swiglu=swiglu, rope=rope, device=device, num_kv_heads=cfg.num_kv_heads)
            for _ in range(cfg.num_layers)])
        for b in self.blocks:
            b.norm1.eps = b.norm2.eps = cfg.norm_eps
            b.attn.theta = cfg.rope_theta
        Norm = RMSNorm if rms else LayerNorm
        self.final_norm = Norm(H, eps=cfg.norm_eps, device=device)
        self.head = None if cfg.tie_embeddings else Linear(H, cfg.vocab_size, bias=False,
                                                           device=device, init_std=cfg.init_std)
        self._pe = None

    def _positions(self, S: int, device):
        if self.cfg.pos != "sinusoidal":
            return None
        if self._pe is None or self._pe.shape[0] < S:
            from ..ops.elementwise import sinusoid_table
            self._pe = sinusoid_table(max(S, self.cfg.max_seq_len), self.cfg.hidden_dim, device)
        return self._pe

    def forward(self, ids: torch.Tensor, targets: Optional[torch.Tensor] = None):
        B, S = ids.shape
        x = F.embedding(ids, self.embed.weight, self._positions(S, ids.device), S)
        for blk in self.blocks:
            x = blk(x, B, S)
        x = self.final_norm(x)
        logits = self.head(x) if self.head is not None else F.linear(
            x, self.embed.weight.t().contiguous())
        if targets is None:
            return logits
        return F.cross_entropy(logits, targets.reshape(-1))

    @torch.no_grad()
    def load_from(self, lm) -> None:
        """Copy the weights of a :class:`DecoderLM` with the same configuration."""
        V = self.cfg.vocab_size
        n1, n2, fn = lm.layout.norm_names
        self.embed.weight.copy_(lm.master["token_embed"][:V])

        def norm(dst, prefix):
            dst.scale.copy_(lm.master[prefix + "_scale"])
            if hasattr(dst, "bias") and dst.bias is not None and (prefix + "_bias") in lm.master:
                dst.bias.copy_(lm.master[prefix + "_bias"])

        for l, b in enumerate(self.blocks):
            p = f"layers.{l}."
            norm(b.norm1, p + n1)
            norm(b.norm2, p + n2)
            b.attn.qkv.weight.copy_(lm.master[p + "attn.qkv_weights"])
            b.attn.o.weight.copy_(lm.master[p + "attn.o_weights"])
            up = "ff.gate_up_weights" if self.cfg.activation == "swiglu" else "ff.up_weights"
            b.mlp.up.weight.copy_(lm.master[p + up])
            b.mlp.down.weight.copy_(lm.master[p + "ff.down_weights"])
            if self.cfg.use_bias:
                b.attn.qkv.bias.copy_(lm.master[p + "attn.qkv_bias"])
                b.attn.o.bias.copy_(lm.master[p + "attn.o_bias"])
                if b.mlp.up.bias is not None:
                    b.mlp.up.bias.copy_(lm.master[p + "ff.up_bias"])
                    b.mlp.down.bias.copy_(lm.master[p + "ff.down_bias"])
        norm(self.final_norm, fn)
        if self.head is not None:
            self.head.weight.copy_(lm.master["output_proj"][:, :V])
