"""Plain PyTorch (autograd, library kernels) restatement of :class:`DecoderLM`.

Used as the numerical oracle for the hand-written forward/backward and as the comparator arm
("the same model on stock PyTorch: cuBLAS GEMMs, SDPA attention, NCCL DDP") of the benchmarks.
It shares the parameter names and ``[in, out]`` weight layout of :mod:`.decoder`.
"""
from __future__ import annotations

from typing import Dict

import torch
import torch.nn.functional as F

from .config import DecoderConfig


def sinusoid(S: int, H: int, device, dtype=torch.float32) -> torch.Tensor:
    pos = torch.arange(S, dtype=torch.float32, device=device)[:, None]
    k = torch.arange(0, H, 2, dtype=torch.float32, device=device)[None, :]
    div = torch.pow(torch.tensor(10000.0, device=device), k / H)
    pe = torch.empty(S, H, dtype=torch.float32, device=device)
    pe[:, 0::2] = torch.sin(pos / div)
    pe[:, 1::2] = torch.cos(pos / div)
    return pe.to(dtype)


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return F.gelu(x, approximate="tanh")


def _rope(x: torch.Tensor, S: int, theta: float) -> torch.Tensor:
    # x: [B, S, nh, dh]; half-split convention
    dh = x.shape[-1]
    half = dh // 2
    pos = torch.arange(S, dtype=torch.float32, device=x.device)
    inv = theta ** (-2.0 * torch.arange(half, dtype=torch.float32, device=x.device) / dh)
    ang = pos[:, None] * inv[None, :]
    sn, cs = torch.sin(ang)[None, :, None, :].to(x.dtype), torch.cos(ang)[None, :, None, :].to(x.dtype)
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * cs - b * sn, a * sn + b * cs], -1)


def forward_logits(params: Dict[str, torch.Tensor], cfg: DecoderConfig,
                   ids: torch.Tensor) -> torch.Tensor:
    """``params`` maps the DecoderLM names to tensors (any float dtype); returns ``[B,S,V]``."""
    B, S = ids.shape
    H, nh, dh = cfg.hidden_dim, cfg.num_heads, cfg.head_dim
    ln = cfg.norm == "layernorm"
    n1n, n2n, fn = ("ln1", "ln2", "final_ln") if ln else ("norm1", "norm2", "final_norm")
    dt = params["token_embed"].dtype

    def norm(x, prefix):
        if ln:
            return F.layer_norm(x, (H,), params[prefix + "_scale"], params[prefix + "_bias"],
                                cfg.norm_eps)
        xf = x.float()
        r = torch.rsqrt((xf * xf).mean(-1, keepdim=True) + cfg.norm_eps)
        return (xf * r).to(x.dtype) * params[prefix + "_scale"]

    x = params["token_embed"][ids]
    if cfg.pos == "sinusoidal":
        x = x + sinusoid(S, H, ids.device, dt)[None]
    for l in range(cfg.num_layers):
        p = f"layers.{l}."
        b = (lambda n: params[p + n]) if cfg.use_bias else (lambda n: None)
        n1 = norm(x, p + n1n)
        qkv = n1 @ params[p + "attn.qkv_weights"]
        if cfg.use_bias:
            qkv = qkv + b("attn.qkv_bias")
        q, k, v = (t.reshape(B, S, nh, dh) for t in qkv.split(H, -1))
        if cfg.pos == "rope":
            q, k = _rope(q, S, cfg.rope_theta), _rope(k, S, cfg.rope_theta)
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                           is_causal=True)
        a = a.transpose(1, 2).reshape(B, S, H)
        o = a @ params[p + "attn.o_weights"]
        if cfg.use_bias:
            o = o + b("attn.o_bias")
        x = x + o
        n2 = norm(x, p + n2n)
        if cfg.activation == "swiglu":
            gu = n2 @ params[p + "ff.gate_up_weights"]
            g, u = gu.split(cfg.intermediate_dim, -1)
            f = (F.silu(g) * u) @ params[p + "ff.down_weights"]
        else:
            u = n2 @ params[p + "ff.up_weights"]
            if cfg.use_bias:
                u = u + b("ff.up_bias")
            f = gelu_tanh(u) @ params[p + "ff.down_weights"]
            if cfg.use_bias:
                f = f + b("ff.down_bias")
        x = x + f
    xf = norm(x, fn)
    if cfg.tie_embeddings:
        return xf @ params["token_embed"].t()
    return xf @ params["output_proj"]


def forward_loss(params: Dict[str, torch.Tensor], cfg: DecoderConfig, ids: torch.Tensor,
                 targets: torch.Tensor) -> torch.Tensor:
    logits = forward_logits(params, cfg, ids)
    loss = F.cross_entropy(logits.reshape(-1, cfg.vocab_size).float(), targets.reshape(-1),
                           ignore_index=-100, reduction="sum")
    return loss / targets.numel()
