"""Typed model configurations.

``Transformer250MConfig`` keeps every field, default and validation message of the reference's
struct (src/core/model.rs:389-550); ``BasicModelConfig`` mirrors src/core/model.rs:283-386.
``DecoderConfig`` is the extended configuration that the GPU model consumes: it adds the choices
the larger configurations need (RMSNorm, RoPE, SwiGLU, mixture of experts) while the reference
values (LayerNorm, sinusoidal positions, tanh-GELU, biases) stay the defaults.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field, replace
from typing import Any, Dict, Optional, Tuple

from ..foundation.error import ConfigError


@dataclass
class BasicModelConfig:
    """src/core/model.rs:283-386 (defaults 512/8/6/512/32000/0.1/1e-5)."""

    model_dim: int = 512
    head_count: int = 8
    layer_count: int = 6
    max_seq_len: int = 512
    vocab_size: int = 32000
    dropout: float = 0.1
    layer_norm_eps: float = 1e-5

    def validate(self) -> None:
        if self.model_dim == 0:
            raise ConfigError.invalid("model_dim", self.model_dim,
                                      "Model dimension must be greater than 0")
        if self.head_count == 0 or self.model_dim % self.head_count != 0:
            raise ConfigError.invalid(
                "model_dim", f"{self.model_dim} (head_count={self.head_count})",
                "Model dimension must be divisible by head count")


@dataclass
class Transformer250MConfig:
    """The reference's transformer configuration (src/core/model.rs:389-423, defaults :534-550).

    The defaults describe a 163,087,441-parameter model (hidden 768, 12 layers); the
    ``benchmark_250m`` preset is the 267,633,920-parameter configuration the benchmarks name.
    """

    hidden_dim: int = 768
    num_layers: int = 12
    num_heads: int = 12
    intermediate_dim: int = 3072
    vocab_size: int = 50257
    max_seq_len: int = 1024
    dropout: float = 0.1
    attention_dropout: float = 0.1
    layer_norm_eps: float = 1e-5
    use_bias: bool = True
    activation: str = "gelu"

    @classmethod
    def new(cls) -> "Transformer250MConfig":
        return cls()

    @classmethod
    def benchmark_250m(cls, max_seq_len: int = 512) -> "Transformer250MConfig":
        return cls(hidden_dim=1024, num_layers=16, num_heads=16, intermediate_dim=4096,
                   vocab_size=32000, max_seq_len=max_seq_len)

    # ModelConfig / VocabularyConfig / SequenceConfig / DropoutConfig accessors
    def model_dim(self) -> int:
        return self.hidden_dim

    def head_count(self) -> int:
        return self.num_heads

    def layer_count(self) -> int:
        return self.num_layers

    def pad_token_id(self) -> Optional[int]:
        return 0

    def use_positional_encoding(self) -> bool:
        return True

    def num_parameters(self) -> int:
        """The config-level estimate (src/core/model.rs:432-484): no output bias."""
        H, I, V, S = self.hidden_dim, self.intermediate_dim, self.vocab_size, self.max_seq_len
        b = 1 if self.use_bias else 0
        per_layer = 3 * H * H + b * 3 * H + H * H + b * H + H * I + b * I + I * H + b * H + 4 * H
        return V * H + S * H + per_layer * self.num_layers + 2 * H + V * H

    def buffer_parameters(self) -> int:
        """Length of the reference's flat parameter buffer, i.e. ``model.num_parameters()``
        (plugins/model-transformer/src/lib.rs:541-580): includes the never-read positional
        table and output bias."""
        H, I, V, S = self.hidden_dim, self.intermediate_dim, self.vocab_size, self.max_seq_len
        n = V * H + S * H
        per = 4 * H * H + 2 * H + H * I + I * H + 2 * H
        if self.use_bias:
            per += 4 * H + I + H
        n += per * self.num_layers + 2 * H + H * V
        if self.use_bias:
            n += V
        return n

    def validate(self) -> None:
        """Union of the reference's two validators with the messages of the inherent one
        (src/core/model.rs:487-531)."""
        if self.hidden_dim == 0:
            raise ConfigError.invalid("hidden_dim", self.hidden_dim,
                                      "Hidden dimension must be greater than 0")
        if self.num_heads == 0 or self.hidden_dim % self.num_heads != 0:
            raise ConfigError.invalid("hidden_dim",
                                      f"{self.hidden_dim} (num_heads={self.num_heads})",
                                      "Hidden dimension must be divisible by number of heads")
        if self.num_layers == 0:
            raise ConfigError.invalid("num_layers", self.num_layers,
                                      "Number of layers must be greater than 0")
        if self.vocab_size == 0:
            raise ConfigError.invalid("vocab_size", self.vocab_size,
                                      "Vocabulary size must be greater than 0")
        if self.max_seq_len == 0:
            raise ConfigError.invalid("max_seq_len", self.max_seq_len,
                                      "Maximum sequence length must be greater than 0")

    def to_decoder(self, **overrides: Any) -> "DecoderConfig":
        cfg = DecoderConfig(
            hidden_dim=self.hidden_dim, num_layers=self.num_layers, num_heads=self.num_heads,
            intermediate_dim=self.intermediate_dim, vocab_size=self.vocab_size,
            max_seq_len=self.max_seq_len, dropout=self.dropout,
            attention_dropout=self.attention_dropout, norm_eps=self.layer_norm_eps,
            use_bias=self.use_bias, activation="gelu", norm="layernorm", pos="sinusoidal")
        return replace(cfg, **overrides)


@dataclass
class DecoderConfig:
    """Configuration of the GPU decoder-only transformer."""

    hidden_dim: int = 768
    num_layers: int = 12
    num_heads: int = 12
    intermediate_dim: int = 3072
    vocab_size: int = 50257
    max_seq_len: int = 1024
    dropout: float = 0.0
    attention_dropout: float = 0.0
    num_kv_heads: int = 0           # grouped-query attention; 0 = one K/V head per query head
    norm_eps: float = 1e-5
    use_bias: bool = True
    activation: str = "gelu"        # "gelu" (tanh approximation) | "swiglu"
    norm: str = "layernorm"         # "layernorm" | "rmsnorm"
    pos: str = "sinusoidal"         # "sinusoidal" | "rope" | "learned" (a trained table) | "none"
    rope_theta: float = 10000.0
    # Llama-3.1 style frequency scaling of the rotary embedding, as a tuple
    # (factor, low_freq_factor, high_freq_factor, original_max_position); None = plain RoPE
    rope_llama3: Optional[Tuple[float, float, float, int]] = None
    num_experts: int = 0            # 0 = dense MLP
    top_k: int = 2
    capacity_factor: float = 1.25
    aux_loss_coef: float = 0.01   # weight of the router load-balancing term
    router_aux_coef: float = 0.01
    tie_embeddings: bool = False
    init_std: float = 0.02

    @property
    def head_dim(self) -> int:
        return self.hidden_dim // self.num_heads

    @property
    def kv_heads(self) -> int:
        return self.num_kv_heads or self.num_heads

    @property
    def kv_dim(self) -> int:
        """Width of the K (and of the V) projection."""
        return self.kv_heads * self.head_dim

    @property
    def qkv_dim(self) -> int:
        return self.hidden_dim + 2 * self.kv_dim

    @property
    def vocab_padded(self) -> int:
        """Vocabulary rounded up to a multiple of 8: the width of the logits buffer and of the
        stored output projection (padding columns stay zero and are ignored by the loss)."""
        return (self.vocab_size + 7) // 8 * 8

    @classmethod
    def transformer_250m(cls, max_seq_len: int = 2048) -> "DecoderConfig":
        # the reference declares dropout = 0.1 in this preset and never applies it (its forward
        # pass has no dropout, plugins/model-transformer/src/lib.rs:791-919); the throughput
        # benchmark trains without dropout, callers that want it pass the rates explicitly
        return Transformer250MConfig.benchmark_250m(max_seq_len).to_decoder(
            dropout=0.0, attention_dropout=0.0)

    @classmethod
    def decoder_1p3b(cls, max_seq_len: int = 4096) -> "DecoderConfig":
        return cls(hidden_dim=2048, num_layers=24, num_heads=16, intermediate_dim=5504,
                   vocab_size=32000, max_seq_len=max_seq_len, use_bias=False,
                   activation="swiglu", norm="rmsnorm", pos="rope")

    @classmethod
    def moe_8x(cls, max_seq_len: int = 2048) -> "DecoderConfig":
        return cls(hidden_dim=2048, num_layers=16, num_heads=16, intermediate_dim=5632,
                   vocab_size=32000, max_seq_len=max_seq_len, use_bias=False,
                   activation="swiglu", norm="rmsnorm", pos="rope", num_experts=8, top_k=2,
                   capacity_factor=1.25)

    def validate(self) -> None:
        Transformer250MConfig(hidden_dim=self.hidden_dim, num_layers=self.num_layers,
                              num_heads=self.num_heads, intermediate_dim=self.intermediate_dim,
                              vocab_size=self.vocab_size, max_seq_len=self.max_seq_len).validate()
        if self.activation not in ("gelu", "swiglu"):
            raise ConfigError.invalid("activation", self.activation,
                                      "Activation must be 'gelu' or 'swiglu'")
        if self.norm not in ("layernorm", "rmsnorm"):
            raise ConfigError.invalid("norm", self.norm, "Norm must be 'layernorm' or 'rmsnorm'")
        if self.pos not in ("sinusoidal", "rope", "none", "learned"):
            raise ConfigError.invalid("pos", self.pos,
                                      "Positions must be 'sinusoidal', 'rope', 'learned' or 'none'")
        if self.hidden_dim % 8 or self.intermediate_dim % 8:
            raise ConfigError.invalid("hidden_dim", self.hidden_dim,
                                      "hidden_dim and intermediate_dim must be multiples of 8 "
                                      "(16-byte rows)")
        if self.num_kv_heads and (self.num_kv_heads < 0 or self.num_heads % self.num_kv_heads):
            raise ConfigError.invalid("num_kv_heads", self.num_kv_heads,
                                      "Key/value heads must divide the number of heads")
        if self.kv_dim % 8:
            raise ConfigError.invalid("num_kv_heads", self.num_kv_heads,
                                      "kv_heads * head_dim must be a multiple of 8 (16-byte rows)")
        for name, rate in (("dropout", self.dropout), ("attention_dropout", self.attention_dropout)):
            # the reference declares the two rates and never applies them (its forward pass is
            # inference only, plugins/model-transformer/src/lib.rs:863-921); here they act in
            # training passes of the decoder (rates are realised in steps of 1/256)
            if not 0.0 <= rate < 1.0:
                raise ConfigError.invalid(name, rate, "Dropout rates must lie in [0, 1)")
        if self.num_experts and not (0 < self.top_k <= self.num_experts):
            raise ConfigError.invalid("top_k", self.top_k, "top_k must be in [1, num_experts]")

    def require_no_dropout(self, where: str) -> None:
        """Dropout is implemented in the single-replica / data-parallel decoder; the other
        execution plans refuse a non-zero rate instead of ignoring it."""
        if self.dropout or self.attention_dropout:
            raise ConfigError.invalid("dropout", self.dropout or self.attention_dropout,
                                      f"Dropout is not implemented under {where}; set dropout "
                                      "and attention_dropout to 0")

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "DecoderConfig":
        known = {f for f in cls.__dataclass_fields__}
        return cls(**{k: v for k, v in d.items() if k in known})
