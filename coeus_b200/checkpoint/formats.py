"""Whole-model checkpoints in three formats.

* ``.rustllm``: the reference's container with its flat parameter layout
  (:mod:`coeus_b200.core.serialization`, :mod:`coeus_b200.models.layout_ref`).
* SafeTensors and GGUF: named tensors.  The reference names the formats only in an enum
  (src/domain/persistence/mod.rs:17-21); tensor names are the reference's field names
  (``token_embed``, ``layers.{l}.ln1_scale``, ``layers.{l}.attn.q_weights`` ...,
  ``layers.{l}.ff.up_weights``, ``final_ln_scale``, ``output_proj``) and weights stay ``[in, out]``
  row-major, not transposed.  File metadata carries the five keys the reference saves
  (``hidden_dim``, ``num_layers``, ``num_heads``, ``vocab_size``, ``max_seq_len``;
  plugins/model-transformer/src/lib.rs:966-971) plus the ones it forgets (``intermediate_dim``,
  ``use_bias``, ``layer_norm_eps``, ``activation`` ...), so a model with a non-default
  feed-forward width reloads with the right layout.

Readers map the file (``numpy.memmap``) and copy tensor by tensor to the device; tensor-parallel
loading slices ``q/k/v/gate/up`` along the output dimension and ``o/down`` along the input
dimension before the copy.
"""
from __future__ import annotations

import os
from typing import Callable, Dict, Optional, Tuple

import numpy as np
import torch

from ..core.serialization import ModelMetadata, read_rustllm, write_rustllm
from ..foundation.error import ProcessingError, invalid_input
from ..models.config import DecoderConfig, Transformer250MConfig
from ..models.layout_ref import (from_reference_flat, load_named_into_model, named_from_model,
                                 reference_offsets, to_reference_flat)
from ..utils import native

_NP = {"F32": np.float32, "F16": np.float16, "I64": np.int64, "I32": np.int32, "U8": np.uint8,
       "F64": np.float64, "BF16": np.uint16}
_TORCH_NAME = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16",
               torch.int64: "I64", torch.int32: "I32", torch.uint8: "U8", torch.float64: "F64"}


def config_metadata(cfg: DecoderConfig) -> Dict[str, str]:
    d = {"architecture": "transformer", "hidden_dim": cfg.hidden_dim, "num_layers": cfg.num_layers,
         "num_heads": cfg.num_heads, "vocab_size": cfg.vocab_size, "max_seq_len": cfg.max_seq_len,
         "intermediate_dim": cfg.intermediate_dim, "use_bias": cfg.use_bias,
         "layer_norm_eps": cfg.norm_eps, "activation": cfg.activation, "dropout": cfg.dropout,
         "attention_dropout": cfg.attention_dropout, "norm": cfg.norm, "pos": cfg.pos,
         "rope_theta": cfg.rope_theta, "num_experts": cfg.num_experts, "top_k": cfg.top_k,
         "capacity_factor": cfg.capacity_factor, "tie_embeddings": cfg.tie_embeddings,
         "num_kv_heads": cfg.num_kv_heads}
    if cfg.rope_llama3 is not None:
        d["rope_llama3"] = ",".join(str(x) for x in cfg.rope_llama3)
    return {k: (str(v).lower() if isinstance(v, bool) else str(v)) for k, v in d.items()}


def _parse_llama3(text):
    if not text:
        return None
    f, lo, hi, orig = text.split(",")
    return float(f), float(lo), float(hi), int(float(orig))


def config_from_metadata(meta: Dict[str, str]) -> DecoderConfig:
    """Missing keys take the reference's defaults (768 / 12 / 12 / 50257 / 1024,
    plugins/model-transformer/src/lib.rs:1067-1099); unknown keys are ignored."""
    base = Transformer250MConfig()

    def geti(k, default):
        return int(meta[k]) if k in meta else default

    def getb(k, default):
        return meta[k].lower() == "true" if k in meta else default

    return DecoderConfig(
        hidden_dim=geti("hidden_dim", base.hidden_dim), num_layers=geti("num_layers", base.num_layers),
        num_heads=geti("num_heads", base.num_heads), vocab_size=geti("vocab_size", base.vocab_size),
        max_seq_len=geti("max_seq_len", base.max_seq_len),
        intermediate_dim=geti("intermediate_dim", base.intermediate_dim),
        use_bias=getb("use_bias", base.use_bias),
        norm_eps=float(meta.get("layer_norm_eps", base.layer_norm_eps)),
        activation=meta.get("activation", "gelu"), dropout=float(meta.get("dropout", 0.0)),
        attention_dropout=float(meta.get("attention_dropout", 0.0)),
        norm=meta.get("norm", "layernorm"), pos=meta.get("pos", "sinusoidal"),
        rope_theta=float(meta.get("rope_theta", 10000.0)), num_experts=geti("num_experts", 0),
        top_k=geti("top_k", 2), capacity_factor=float(meta.get("capacity_factor", 1.25)),
        tie_embeddings=getb("tie_embeddings", False), num_kv_heads=geti("num_kv_heads", 0),
        rope_llama3=_parse_llama3(meta.get("rope_llama3")))


# ------------------------------------------------------------------------------ named tensors
def _as_numpy(t: torch.Tensor) -> Tuple[np.ndarray, str]:
    t = t.detach().to("cpu").contiguous()
    name = _TORCH_NAME[t.dtype]
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16), name
    return t.numpy(), name


def save_safetensors(path: str, tensors: Dict[str, torch.Tensor],
                     metadata: Optional[Dict[str, str]] = None) -> None:
    items, keep = [], []
    for name in sorted(tensors):
        arr, dt = _as_numpy(tensors[name])
        keep.append(arr)
        items.append((name, dt, list(tensors[name].shape), arr.reshape(-1)))
    native.module().safetensors_write(path, items, dict(metadata or {}))


def save_gguf(path: str, tensors: Dict[str, torch.Tensor],
              metadata: Optional[Dict[str, str]] = None) -> None:
    items, keep = [], []
    for name in sorted(tensors):
        arr, dt = _as_numpy(tensors[name])
        keep.append(arr)
        items.append((name, dt, list(tensors[name].shape), arr.reshape(-1)))
    meta = {"general.architecture": "transformer"}
    for k, v in (metadata or {}).items():
        meta[k if k.startswith("general.") else f"rustllm.{k}"] = v
    native.module().gguf_write(path, items, meta)


def _load_indexed(path: str, index: dict, names=None, slicer=None) -> Dict[str, torch.Tensor]:
    mm = np.memmap(path, dtype=np.uint8, mode="r")
    out = {}
    for t in index["tensors"]:
        if names is not None and t["name"] not in names:
            continue
        raw = mm[t["offset"]:t["offset"] + t["nbytes"]]
        arr = np.frombuffer(raw, dtype=_NP[t["dtype"]]).reshape(t["shape"])
        if slicer is not None:
            arr = slicer(t["name"], arr)
        ten = torch.from_numpy(np.array(arr, copy=True))
        if t["dtype"] == "BF16":
            ten = ten.view(torch.int16).view(torch.bfloat16)
        out[t["name"]] = ten
    return out


def load_safetensors(path: str, names=None, slicer=None
                     ) -> Tuple[Dict[str, torch.Tensor], Dict[str, str]]:
    try:
        index = native.module().safetensors_index(path)
    except ValueError as e:
        raise invalid_input(str(e)) from None
    return _load_indexed(path, index, names, slicer), dict(index["metadata"])


def load_gguf(path: str, names=None, slicer=None) -> Tuple[Dict[str, torch.Tensor], Dict[str, str]]:
    try:
        index = native.module().gguf_index(path)
    except ValueError as e:
        raise invalid_input(str(e)) from None
    meta = {(k[len("rustllm."):] if k.startswith("rustllm.") else k): v
            for k, v in index["metadata"].items()}
    return _load_indexed(path, index, names, slicer), meta


def tp_slicer(cfg: DecoderConfig, tp_rank: int, tp_size: int):
    """Slices reference-named tensors for one tensor-parallel rank: ``q/k/v/gate/up`` (and their
    biases) along the output dimension, ``o/down`` along the input dimension, ``token_embed`` and
    ``output_proj`` along the vocabulary."""
    def cut(a, dim):
        n = a.shape[dim] // tp_size
        idx = [slice(None)] * a.ndim
        idx[dim] = slice(tp_rank * n, (tp_rank + 1) * n)
        return a[tuple(idx)]

    def slicer(name: str, arr):
        leaf = name.split(".")[-1]
        if leaf in ("q_weights", "k_weights", "v_weights", "up_weights", "gate_weights"):
            return cut(arr, 1)
        if leaf in ("q_bias", "k_bias", "v_bias", "up_bias"):
            return cut(arr, 0)
        if leaf in ("o_weights", "down_weights"):
            return cut(arr, 0)
        if name == "token_embed":
            return cut(arr, 0)
        if name == "output_proj":
            return cut(arr, 1)
        return arr
    return slicer


# ------------------------------------------------------------------------------ whole models
def save_model(model, path: str, fmt: Optional[str] = None,
               progress: Optional[Callable[[int, int], None]] = None,
               tail: Optional[torch.Tensor] = None) -> None:
    """``fmt``: ``rustllm`` | ``safetensors`` | ``gguf`` (default: from the file extension)."""
    fmt = fmt or os.path.splitext(path)[1].lstrip(".").lower()
    named = named_from_model(model)
    meta = config_metadata(model.cfg)
    if fmt == "rustllm":
        if model.cfg.kv_heads != model.cfg.num_heads:
            raise ProcessingError.unsupported(
                "grouped-query attention in a .rustllm file",
                "the reference's flat layout has square K and V projections")
        flat = to_reference_flat(named, model.cfg)
        if tail is not None:
            flat[flat.numel() - tail.numel():] = tail.to(torch.float32).cpu()
        md = ModelMetadata.new("transformer")
        for k in ("hidden_dim", "num_layers", "num_heads", "vocab_size", "max_seq_len"):
            md.with_custom(k, meta[k])
        for k, v in meta.items():
            if k not in ("architecture", "hidden_dim", "num_layers", "num_heads", "vocab_size",
                         "max_seq_len"):
                md.with_custom(k, v)
        write_rustllm(path, flat.numpy(), md, progress)
    elif fmt == "safetensors":
        save_safetensors(path, named, meta)
    elif fmt == "gguf":
        save_gguf(path, named, meta)
    else:
        raise ProcessingError.unsupported(f"Loading file format: {path}")


def load_model(path: str, device="cuda", fmt: Optional[str] = None, training: bool = False,
               progress: Optional[Callable[[int, int], None]] = None):
    """Returns ``(DecoderLM, tail)``; ``tail`` is the unread remainder of a ``.rustllm`` buffer
    (kept so that saving again reproduces the file byte for byte), else ``None``."""
    from ..models.decoder import DecoderLM
    fmt = fmt or os.path.splitext(path)[1].lstrip(".").lower()
    tail = None
    if fmt == "rustllm":
        _, params, md = read_rustllm(path, progress)
        cfg = config_from_metadata(dict(md.custom))
        flat = torch.from_numpy(np.array(params, dtype=np.float32, copy=True))
        named = from_reference_flat(flat, cfg)
        used = sum(int(np.prod(s)) for _, s in reference_offsets(cfg).values())
        tail = flat[used:].clone()
    elif fmt == "safetensors":
        named, meta = load_safetensors(path)
        cfg = config_from_metadata(meta)
    elif fmt == "gguf":
        named, meta = load_gguf(path)
        cfg = config_from_metadata(meta)
    else:
        raise ProcessingError.unsupported(f"Loading file format: {path}")
    dev = torch.device(device)
    model = DecoderLM(cfg, device=dev, init="zeros", training=training,
                      dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32)
    load_named_into_model(model, named)
    return model, tail
