"""Llama-style checkpoints in the Hugging Face tensor naming (``model.layers.N.self_attn.q_proj
.weight`` ..., weights stored ``[out, in]``) to and from the decoder of this framework (weights
``[in, out]``, q/k/v fused, gate and up fused).  Covers the multi-head-attention members of the
family and the grouped-query ones (fewer key/value heads; the attention kernels are multi-head,
so K and V are expanded per group before they run).
Mixtral-style mixtures of experts load too (router ``mlp.gate``, fused ``mlp.experts.gate_up_proj``
/ ``down_proj``), with a capacity that never drops a token.
The reference has its own flat ``.rustllm`` layout only (src/core/serialization.rs) and names
SafeTensors / GGUF as formats without reading them (src/domain/persistence/mod.rs:20-24)."""
from __future__ import annotations

from typing import Any, Dict, Mapping, Tuple

import torch

from ..foundation.error import ProcessingError
from ..models.config import DecoderConfig


def _get(cfg: Any, key: str, default=None):
    return cfg.get(key, default) if isinstance(cfg, Mapping) else getattr(cfg, key, default)


def config_from_hf(hf_config: Any) -> DecoderConfig:
    """``hf_config``: a ``LlamaConfig``-like object or the dict of its ``config.json``."""
    nh = _get(hf_config, "num_attention_heads")
    nkv = _get(hf_config, "num_key_value_heads", nh) or nh
    if nh % nkv:
        raise ProcessingError.invalid_input(f"{nkv} key/value heads do not divide {nh} heads")
    if _get(hf_config, "mlp_bias", False):
        raise ProcessingError.unsupported("feed-forward biases in a Llama-style checkpoint",
                                          "the SwiGLU path has none")
    # Qwen2-style checkpoints carry q/k/v biases (and no output-projection bias)
    attn_bias = bool(_get(hf_config, "attention_bias", False)) or \
        _get(hf_config, "model_type", "") == "qwen2"
    scaling = _get(hf_config, "rope_scaling", None) or _get(hf_config, "rope_parameters", None)
    kind = _get(scaling, "rope_type", _get(scaling, "type", "default")) if scaling else "default"
    llama3 = None
    if kind == "llama3":
        llama3 = (float(_get(scaling, "factor")), float(_get(scaling, "low_freq_factor")),
                  float(_get(scaling, "high_freq_factor")),
                  int(_get(scaling, "original_max_position_embeddings")))
    elif kind not in ("default", None):
        raise ProcessingError.unsupported(f"rotary scaling '{kind}'", "plain and llama3 only")
    window = _get(hf_config, "sliding_window", None)
    if _get(hf_config, "use_sliding_window", True) is False:
        window = None
    if window and window < _get(hf_config, "max_position_embeddings", 0):
        raise ProcessingError.unsupported(f"sliding-window attention (window {window})",
                                          "the attention kernels are fully causal")
    act = _get(hf_config, "hidden_act", "silu")
    if act != "silu":
        raise ProcessingError.unsupported(f"activation '{act}'", "SwiGLU uses SiLU")
    theta = _get(hf_config, "rope_theta", None)
    if theta is None and _get(hf_config, "rope_parameters", None):
        theta = _get(_get(hf_config, "rope_parameters"), "rope_theta", 10000.0)
    experts = int(_get(hf_config, "num_local_experts", 0) or 0)
    moe = {}
    if experts:
        # Mixtral-style routing has no capacity limit; a capacity factor of E / k reserves room
        # for every token at every expert, so nothing is ever dropped
        k = int(_get(hf_config, "num_experts_per_tok", 2))
        moe = dict(num_experts=experts, top_k=k, capacity_factor=float(experts) / k,
                   aux_loss_coef=float(_get(hf_config, "router_aux_loss_coef", 0.0) or 0.0))
    return DecoderConfig(
        **moe,
        hidden_dim=_get(hf_config, "hidden_size"), num_layers=_get(hf_config, "num_hidden_layers"),
        num_heads=nh, num_kv_heads=0 if nkv == nh else nkv, intermediate_dim=_get(hf_config, "intermediate_size"),
        vocab_size=_get(hf_config, "vocab_size"),
        max_seq_len=_get(hf_config, "max_position_embeddings", 2048),
        norm_eps=float(_get(hf_config, "rms_norm_eps", 1e-6)), use_bias=attn_bias,
        activation="swiglu", norm="rmsnorm", pos="rope", rope_theta=float(theta or 10000.0),
        rope_llama3=llama3,
        tie_embeddings=bool(_get(hf_config, "tie_word_embeddings", False)))


def load_hf_llama(state: Mapping[str, torch.Tensor], hf_config: Any, device="cuda",
                  training: bool = False):
    """A :class:`coeus_b200.models.decoder.DecoderLM` holding the weights of ``state``."""
    from ..models.decoder import DecoderLM
    cfg = config_from_hf(hf_config)
    dev = torch.device(device)
    lm = DecoderLM(cfg, dev, init="zeros", training=training,
                   dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32)
    V = cfg.vocab_size
    n1, n2, fn = lm.layout.norm_names

    def t(name: str) -> torch.Tensor:
        if name not in state:
            raise ProcessingError.invalid_input(f"missing tensor '{name}'")
        return state[name].to(torch.float32)

    lm.master["token_embed"][:V] = t("model.embed_tokens.weight")
    for l in range(cfg.num_layers):
        h, p = f"model.layers.{l}.", f"layers.{l}."
        lm.master[p + "attn.qkv_weights"].copy_(torch.cat(
            [t(h + f"self_attn.{x}_proj.weight").t() for x in ("q", "k", "v")], 1))
        lm.master[p + "attn.o_weights"].copy_(t(h + "self_attn.o_proj.weight").t())
        if cfg.use_bias:
            lm.master[p + "attn.qkv_bias"].copy_(torch.cat(
                [t(h + f"self_attn.{x}_proj.bias") for x in ("q", "k", "v")]))
            if h + "self_attn.o_proj.bias" in state:
                lm.master[p + "attn.o_bias"].copy_(t(h + "self_attn.o_proj.bias"))
        if cfg.num_experts:
            # Mixtral naming: router [E, H]; experts fused as gate_up [E, 2I, H], down [E, H, I]
            lm.master[p + "moe.router_weights"].copy_(t(h + "mlp.gate.weight").t())
            lm.master[p + "moe.experts.gate_up_weights"].copy_(
                t(h + "mlp.experts.gate_up_proj").transpose(1, 2))
            lm.master[p + "moe.experts.down_weights"].copy_(
                t(h + "mlp.experts.down_proj").transpose(1, 2))
        else:
            lm.master[p + "ff.gate_up_weights"].copy_(torch.cat(
                [t(h + "mlp.gate_proj.weight").t(), t(h + "mlp.up_proj.weight").t()], 1))
            lm.master[p + "ff.down_weights"].copy_(t(h + "mlp.down_proj.weight").t())
        lm.master[p + n1 + "_scale"].copy_(t(h + "input_layernorm.weight"))
        lm.master[p + n2 + "_scale"].copy_(t(h + "post_attention_layernorm.weight"))
    lm.master[fn + "_scale"].copy_(t("model.norm.weight"))
    if not cfg.tie_embeddings:
        lm.master["output_proj"][:, :V] = t("lm_head.weight").t()
    lm.sync_working_copy()
    return lm


def config_from_hf_gpt2(hf_config: Any) -> DecoderConfig:
    """GPT-2 family: LayerNorm, tanh-GELU, biases everywhere, a trained position table, and the
    output projection tied to the token embedding."""
    act = _get(hf_config, "activation_function", "gelu_new")
    if act not in ("gelu_new", "gelu_pytorch_tanh"):
        raise ProcessingError.unsupported(f"activation '{act}'", "the GELU kernel is the tanh form")
    if _get(hf_config, "scale_attn_by_inverse_layer_idx", False) or \
            _get(hf_config, "reorder_and_upcast_attn", False):
        raise ProcessingError.unsupported("per-layer attention scaling", "1/sqrt(head_dim) only")
    H = _get(hf_config, "n_embd")
    return DecoderConfig(
        hidden_dim=H, num_layers=_get(hf_config, "n_layer"), num_heads=_get(hf_config, "n_head"),
        intermediate_dim=_get(hf_config, "n_inner", None) or 4 * H,
        vocab_size=_get(hf_config, "vocab_size"), max_seq_len=_get(hf_config, "n_positions", 1024),
        norm_eps=float(_get(hf_config, "layer_norm_epsilon", 1e-5)), use_bias=True,
        activation="gelu", norm="layernorm", pos="learned",
        tie_embeddings=bool(_get(hf_config, "tie_word_embeddings", True)))


def load_hf_gpt2(state: Mapping[str, torch.Tensor], hf_config: Any, device="cuda",
                 training: bool = False):
    """A :class:`coeus_b200.models.decoder.DecoderLM` holding a ``GPT2LMHeadModel`` state dict.
    GPT-2 stores its projections as ``[in, out]`` already (its ``Conv1D``), which is the layout
    used here, so nothing is transposed."""
    from ..models.decoder import DecoderLM
    cfg = config_from_hf_gpt2(hf_config)
    dev = torch.device(device)
    lm = DecoderLM(cfg, dev, init="zeros", training=training,
                   dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32)
    V = cfg.vocab_size
    n1, n2, fn = lm.layout.norm_names

    def t(name: str) -> torch.Tensor:
        for k in (name, "transformer." + name):
            if k in state:
                return state[k].to(torch.float32)
        raise ProcessingError.invalid_input(f"missing tensor '{name}'")

    lm.master["token_embed"][:V] = t("wte.weight")
    lm.master["pos_embed"].copy_(t("wpe.weight"))
    for l in range(cfg.num_layers):
        h, p = f"h.{l}.", f"layers.{l}."
        for ours, theirs in (("attn.qkv", "attn.c_attn"), ("attn.o", "attn.c_proj"),
                             ("ff.up", "mlp.c_fc"), ("ff.down", "mlp.c_proj")):
            lm.master[p + ours + "_weights"].copy_(t(h + theirs + ".weight"))
            lm.master[p + ours + "_bias"].copy_(t(h + theirs + ".bias"))
        for ours, theirs in ((n1, "ln_1"), (n2, "ln_2")):
            lm.master[p + ours + "_scale"].copy_(t(h + theirs + ".weight"))
            lm.master[p + ours + "_bias"].copy_(t(h + theirs + ".bias"))
    lm.master[fn + "_scale"].copy_(t("ln_f.weight"))
    lm.master[fn + "_bias"].copy_(t("ln_f.bias"))
    if not cfg.tie_embeddings:
        lm.master["output_proj"][:, :V] = state["lm_head.weight"].to(torch.float32).t()
    lm.sync_working_copy()
    return lm


def to_hf_gpt2(lm) -> Tuple[Dict[str, torch.Tensor], Dict[str, Any]]:
    """``(state dict, config.json fields)`` of a ``GPT2LMHeadModel`` for a model of that family
    (LayerNorm, tanh-GELU, biases, learned positions, tied head)."""
    cfg = lm.cfg
    if not (cfg.pos == "learned" and cfg.norm == "layernorm" and cfg.activation == "gelu"
            and cfg.use_bias and cfg.tie_embeddings and not cfg.num_experts
            and cfg.kv_heads == cfg.num_heads):
        raise ProcessingError.unsupported("export of this configuration in the GPT-2 naming",
                                          "LayerNorm, GELU, biases, learned positions and a "
                                          "tied head are that family")
    V = cfg.vocab_size
    n1, n2, fn = lm.layout.norm_names
    m = lm.master
    out: Dict[str, torch.Tensor] = {"transformer.wte.weight": m["token_embed"][:V].clone(),
                                    "transformer.wpe.weight": m["pos_embed"].clone()}
    for l in range(cfg.num_layers):
        h, p = f"transformer.h.{l}.", f"layers.{l}."
        for ours, theirs in (("attn.qkv", "attn.c_attn"), ("attn.o", "attn.c_proj"),
                             ("ff.up", "mlp.c_fc"), ("ff.down", "mlp.c_proj")):
            out[h + theirs + ".weight"] = m[p + ours + "_weights"].clone()
            out[h + theirs + ".bias"] = m[p + ours + "_bias"].clone()
        for ours, theirs in ((n1, "ln_1"), (n2, "ln_2")):
            out[h + theirs + ".weight"] = m[p + ours + "_scale"].clone()
            out[h + theirs + ".bias"] = m[p + ours + "_bias"].clone()
    out["transformer.ln_f.weight"] = m[fn + "_scale"].clone()
    out["transformer.ln_f.bias"] = m[fn + "_bias"].clone()
    hf = {"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "n_embd": cfg.hidden_dim,
          "n_layer": cfg.num_layers, "n_head": cfg.num_heads, "n_inner": cfg.intermediate_dim,
          "n_positions": cfg.max_seq_len, "vocab_size": V,
          "layer_norm_epsilon": cfg.norm_eps, "activation_function": "gelu_new",
          "resid_pdrop": 0.0, "embd_pdrop": 0.0, "attn_pdrop": 0.0,
          "tie_word_embeddings": True, "torch_dtype": "float32"}
    return out, hf


def to_hf_llama(lm) -> Tuple[Dict[str, torch.Tensor], Dict[str, Any]]:
    """``(state dict in the Hugging Face naming, config.json fields)`` of a Llama-style
    :class:`DecoderLM` (RMSNorm, SwiGLU, RoPE, no biases, dense)."""
    cfg = lm.cfg
    if not (cfg.norm == "rmsnorm" and cfg.activation == "swiglu" and cfg.pos == "rope"
            and not cfg.use_bias and not cfg.num_experts):
        raise ProcessingError.unsupported("export of a non-Llama-style decoder",
                                          "needs RMSNorm, SwiGLU, RoPE, no biases, no experts")
    H, I, V = cfg.hidden_dim, cfg.intermediate_dim, cfg.vocab_size
    n1, n2, fn = lm.layout.norm_names
    m = lm.master
    out: Dict[str, torch.Tensor] = {"model.embed_tokens.weight": m["token_embed"][:V].clone()}
    for l in range(cfg.num_layers):
        h, p = f"model.layers.{l}.", f"layers.{l}."
        qkv = m[p + "attn.qkv_weights"]
        Hkv = cfg.kv_dim
        for x, lo, hi in (("q", 0, H), ("k", H, H + Hkv), ("v", H + Hkv, H + 2 * Hkv)):
            out[h + f"self_attn.{x}_proj.weight"] = qkv[:, lo:hi].t().contiguous()
        out[h + "self_attn.o_proj.weight"] = m[p + "attn.o_weights"].t().contiguous()
        gu = m[p + "ff.gate_up_weights"]
        out[h + "mlp.gate_proj.weight"] = gu[:, :I].t().contiguous()
        out[h + "mlp.up_proj.weight"] = gu[:, I:].t().contiguous()
        out[h + "mlp.down_proj.weight"] = m[p + "ff.down_weights"].t().contiguous()
        out[h + "input_layernorm.weight"] = m[p + n1 + "_scale"].clone()
        out[h + "post_attention_layernorm.weight"] = m[p + n2 + "_scale"].clone()
    out["model.norm.weight"] = m[fn + "_scale"].clone()
    if not cfg.tie_embeddings:
        out["lm_head.weight"] = m["output_proj"][:, :V].t().contiguous()
    hf = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": H,
          "intermediate_size": I, "num_hidden_layers": cfg.num_layers,
          "num_attention_heads": cfg.num_heads, "num_key_value_heads": cfg.kv_heads,
          "vocab_size": V, "max_position_embeddings": cfg.max_seq_len,
          "rms_norm_eps": cfg.norm_eps, "rope_theta": cfg.rope_theta, "hidden_act": "silu",
          "tie_word_embeddings": cfg.tie_embeddings, "attention_bias": False, "mlp_bias": False}
    if cfg.rope_llama3 is not None:
        f, lo, hi, orig = cfg.rope_llama3
        hf["rope_scaling"] = {"rope_type": "llama3", "factor": f, "low_freq_factor": lo,
                              "high_freq_factor": hi, "original_max_position_embeddings": orig}
    return out, hf


def load_hf_dir(path: str, device="cuda", training: bool = False):
    """A model directory in the Hugging Face layout: ``config.json`` plus one ``.safetensors``
    file or several with ``model.safetensors.index.json``."""
    import glob
    import json
    import os

    from .formats import load_safetensors
    with open(os.path.join(path, "config.json")) as f:
        hf_config = json.load(f)
    files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if not files:
        raise ProcessingError.invalid_input(f"no .safetensors file in {path}")
    state: Dict[str, torch.Tensor] = {}
    for fpath in files:
        tensors, _ = load_safetensors(fpath)
        state.update(tensors)
    if hf_config.get("model_type") == "gpt2":
        return load_hf_gpt2(state, hf_config, device=device, training=training)
    return load_hf_llama(state, hf_config, device=device, training=training)


def save_hf_dir(lm, path: str) -> None:
    """Write ``config.json`` and ``model.safetensors`` in the Hugging Face naming."""
    import json
    import os

    from .formats import save_safetensors
    os.makedirs(path, exist_ok=True)
    state, fields = to_hf_gpt2(lm) if lm.cfg.pos == "learned" else to_hf_llama(lm)
    save_safetensors(os.path.join(path, "model.safetensors"), state, {"format": "pt"})
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(fields, f, indent=1)
