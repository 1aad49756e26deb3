"""The reference's flat parameter layout and its tensor names.

The reference keeps every parameter in one flat ``Vec<f32>`` and slices it by offset
(plugins/model-transformer/src/lib.rs:677-740 for the offsets, :838-880 and :903-916 for the
per-layer order).  It has no tensor names; the names here are its field and local-variable names
(``token_embed``, ``ln1_scale``, ``q_weights`` ... ``output_proj``).  ``reference_offsets`` maps
each name to ``(offset, shape)`` in that buffer, ``to_reference_flat`` / ``from_reference_flat``
convert between the buffer and a dict of named tensors, and ``named_from_model`` /
``load_named_into_model`` translate to and from the GPU model's fused layout.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, Tuple

import torch

from ..foundation.error import ProcessingError
from .config import DecoderConfig


def reference_offsets(cfg: DecoderConfig) -> "OrderedDict[str, Tuple[int, Tuple[int, ...]]]":
    """Offsets follow the reference exactly for its architecture (LayerNorm, GELU, q/k/v/o);
    layer-norm biases are always present there, linear biases only with ``use_bias``."""
    H, I, V, L = cfg.hidden_dim, cfg.intermediate_dim, cfg.vocab_size, cfg.num_layers
    out: "OrderedDict[str, Tuple[int, Tuple[int, ...]]]" = OrderedDict()
    off = 0

    def add(name, shape):
        nonlocal off
        n = 1
        for s in shape:
            n *= s
        out[name] = (off, tuple(shape))
        off += n

    ln = cfg.norm == "layernorm"
    add("token_embed", (V, H))
    for l in range(L):
        p = f"layers.{l}."
        add(p + ("ln1_scale" if ln else "norm1_scale"), (H,))
        if ln:
            add(p + "ln1_bias", (H,))
        for part in ("q", "k", "v", "o"):
            add(p + f"attn.{part}_weights", (H, H))
        if cfg.use_bias:
            for part in ("q", "k", "v", "o"):
                add(p + f"attn.{part}_bias", (H,))
        add(p + ("ln2_scale" if ln else "norm2_scale"), (H,))
        if ln:
            add(p + "ln2_bias", (H,))
        if cfg.num_experts:
            add(p + "moe.router_weights", (H, cfg.num_experts))
            add(p + "moe.experts.gate_up_weights", (cfg.num_experts, H, 2 * I))
            add(p + "moe.experts.down_weights", (cfg.num_experts, I, H))
        elif cfg.activation == "swiglu":
            add(p + "ff.gate_up_weights", (H, 2 * I))
            add(p + "ff.down_weights", (I, H))
        else:
            add(p + "ff.up_weights", (H, I))
            add(p + "ff.down_weights", (I, H))
            if cfg.use_bias:
                add(p + "ff.up_bias", (I,))
                add(p + "ff.down_bias", (H,))
    add("final_ln_scale" if ln else "final_norm_scale", (H,))
    if ln:
        add("final_ln_bias", (H,))
    if not cfg.tie_embeddings:
        add("output_proj", (H, V))
    return out


def reference_buffer_len(cfg: DecoderConfig) -> int:
    """Length of the reference's buffer: the tensors read by ``forward`` plus the tail it
    allocates and serialises but never reads (``max_seq_len * H`` positional slots and, with
    ``use_bias``, ``V`` output-bias slots; lib.rs:541-580)."""
    offs = reference_offsets(cfg)
    last_off, last_shape = next(reversed(offs.values()))
    n = 1
    for s in last_shape:
        n *= s
    used = last_off + n
    tail = cfg.max_seq_len * cfg.hidden_dim + (cfg.vocab_size if cfg.use_bias else 0)
    return used + tail


def to_reference_flat(named: Dict[str, torch.Tensor], cfg: DecoderConfig,
                      tail_fill: float = 0.0) -> torch.Tensor:
    flat = torch.full((reference_buffer_len(cfg),), tail_fill, dtype=torch.float32)
    for name, (off, shape) in reference_offsets(cfg).items():
        if name not in named:
            raise ProcessingError.invalid_input(f"missing tensor '{name}'")
        t = named[name].detach().to("cpu", torch.float32).reshape(-1)
        flat[off:off + t.numel()] = t
    return flat


def from_reference_flat(flat: torch.Tensor, cfg: DecoderConfig) -> Dict[str, torch.Tensor]:
    need = reference_buffer_len(cfg)
    if flat.numel() < need - (cfg.max_seq_len * cfg.hidden_dim
                              + (cfg.vocab_size if cfg.use_bias else 0)):
        raise ProcessingError.shape_mismatch(f"[{need}]", f"[{flat.numel()}]")
    out = {}
    for name, (off, shape) in reference_offsets(cfg).items():
        n = 1
        for s in shape:
            n *= s
        out[name] = flat[off:off + n].view(shape)
    return out


def named_from_model(model) -> Dict[str, torch.Tensor]:
    """Reference-named fp32 tensors (q/k/v split out of the fused matrix) of a DecoderLM."""
    cfg = model.cfg
    H = cfg.hidden_dim
    Hkv = getattr(cfg, "kv_dim", H)
    spans = (("q", 0, H), ("k", H, H + Hkv), ("v", H + Hkv, H + 2 * Hkv))
    out: Dict[str, torch.Tensor] = {}
    for name, t in model.named_parameters():
        if name.endswith("attn.qkv_weights"):
            for part, lo, hi in spans:
                out[name.replace("qkv_weights", f"{part}_weights")] = t[:, lo:hi].contiguous()
        elif name.endswith("attn.qkv_bias"):
            for part, lo, hi in spans:
                out[name.replace("qkv_bias", f"{part}_bias")] = t[lo:hi].contiguous()
        elif name == "output_proj":
            out[name] = t[:, :cfg.vocab_size].contiguous()
        elif name == "token_embed":
            out[name] = t[:cfg.vocab_size].contiguous()
        else:
            out[name] = t
    return out


def load_named_into_model(model, named: Dict[str, torch.Tensor]) -> None:
    expected = set(named_from_model(model).keys())
    missing = expected - set(named.keys())
    if missing:
        raise ProcessingError.invalid_input(f"missing tensors: {sorted(missing)[:4]}...")
    for name in expected:
        model._assign_reference_tensor(name, named[name].to(model.device, torch.float32))
    model.sync_working_copy()
