"""Transformer model plugin (plugins/model-transformer/src/lib.rs): identity
``transformer_model`` v0.1.0, features ``model_building, transformer, 250M_params``;
``create_builder().build(config)`` validates the configuration, allocates the parameters with the
reference's deterministic sin-init and returns a model whose ``forward(ids)`` yields the logits of
the last position (length ``vocab_size``), ``num_parameters()`` the length of the reference's flat
buffer (163,087,441 for the default configuration) and ``write_to`` / ``read_from`` the
``.rustllm`` container.  The compute runs through :class:`coeus_b200.models.decoder.DecoderLM`
(hand-written sm_100a kernels on a GPU, the ops' fp32 oracle on CPU).  Extensions over the
reference: ``forward_batch`` (all positions of a batch), ``generate`` (greedy / temperature /
top-k / top-p with a KV cache), ``save`` / ``load`` in SafeTensors and GGUF, and training through
:class:`coeus_b200.train.Trainer`."""
from __future__ import annotations

import io
import os
from typing import BinaryIO, List, Optional, Sequence, Union

import torch

from ...core.model import (BasicGenerationConfig, BatchedModel, GenerativeModel, ModelBuilder,
                           QuantizableModel)
from ...core.plugin import ModelBuilderPlugin, PluginCapabilities
from ...core.serialization import (ModelMetadata, ModelSerializable, read_rustllm_stream,
                                   write_rustllm_stream)
from ...foundation.error import ProcessingError, invalid_input
from ...foundation.types import Version
from ...models.config import DecoderConfig, Transformer250MConfig
from ...models.decoder import DecoderLM
from ...models.layout_ref import (from_reference_flat, load_named_into_model, named_from_model,
                                  reference_buffer_len, reference_offsets, to_reference_flat)


def _default_device(device: str = "auto") -> torch.device:
    if device != "auto":
        return torch.device(device)
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() \
        else torch.device("cpu")


from . import transformer_math as math  # noqa: E402  (the plugin's `mod math`)

class TransformerModel(GenerativeModel, BatchedModel, ModelSerializable, QuantizableModel):
    def __init__(self, config: Union[Transformer250MConfig, DecoderConfig], lm: DecoderLM,
                 tail: Optional[torch.Tensor] = None, init: str = "reference") -> None:
        self._config = config
        self.lm = lm
        self._tail = tail
        self._init = init
        self._engine = None
        self._quant = None

    # ---- Model / ForwardModel
    def config(self):
        return self._config

    def name(self) -> str:
        return "TransformerModel"

    def decoder_config(self) -> DecoderConfig:
        return self.lm.cfg

    # ---- QuantizableModel (src/core/model.rs:191-200)
    def quantize(self, config=None) -> None:
        """Weight-only quantisation in place (see :mod:`coeus_b200.models.quant`); the codes and
        scales stay available as ``quantized_tensors``."""
        from ...models.quant import QuantConfig, quantize_model_
        cfg = config or QuantConfig()
        self.quantized_tensors = quantize_model_(self.lm, cfg)
        self._quant = cfg
        self._engine = None

    def is_quantized(self) -> bool:
        return self._quant is not None

    def num_parameters(self) -> int:
        return reference_buffer_len(self.lm.cfg)

    def _ids_tensor(self, ids: Sequence[int]) -> torch.Tensor:
        V = self.lm.cfg.vocab_size
        t = torch.as_tensor(ids, dtype=torch.int64)
        if t.numel():
            bad = (t < 0) | (t >= V)
            if bool(bad.any()):
                first = int(t.reshape(-1)[bad.reshape(-1)][0])
                raise invalid_input(f"Token ID {first} out of range [0, {V - 1}]")
        return t.to(self.lm.device)

    def forward(self, input: Sequence[int]) -> List[float]:
        """Logits of the last position for one sequence of token ids."""
        ids = self._ids_tensor(input)
        if ids.dim() != 1:
            raise invalid_input("forward takes one sequence; use forward_batch for [B, S]")
        if ids.numel() == 0:
            raise invalid_input(f"Sequence length 0 out of range [1, {self.lm.cfg.max_seq_len}]")
        logits = self.lm.forward_logits(ids[None], last_only=True)
        return logits[0].float().cpu().tolist()

    def forward_batch(self, batch) -> torch.Tensor:
        """Logits ``[B, S, V]`` for a batch of equally long sequences."""
        ids = self._ids_tensor(batch)
        if ids.dim() == 1:
            ids = ids[None]
        return self.lm.forward_logits(ids)

    def generate(self, input: Sequence[int], config: Optional[BasicGenerationConfig] = None,
                 seed: int = 0) -> List[int]:
        """Continues ``input`` until ``config.max_length`` tokens in total."""
        from ...infer.engine import InferenceEngine
        if self._engine is None:
            self._engine = InferenceEngine(self.lm)
        cfg = config or BasicGenerationConfig()
        ids = self._ids_tensor(input)
        n_new = max(0, cfg.max_length - ids.numel())
        out = self._engine.generate(ids[None], max_new_tokens=n_new, temperature=cfg.temperature,
                                    top_k=cfg.top_k, top_p=cfg.top_p, seed=seed)
        return out[0].tolist()

    # ---- ModelSerializable
    def _reference_flat(self) -> torch.Tensor:
        cfg = self.lm.cfg
        flat = to_reference_flat(named_from_model(self.lm), cfg)
        used = sum(int(torch.Size(s).numel()) for _, s in reference_offsets(cfg).values())
        if self._tail is not None:
            flat[used:] = self._tail.to(torch.float32).cpu()
        elif self._init == "reference" and flat.numel() > used:
            from ...ops.elementwise import sin_init_
            tail = torch.empty(flat.numel() - used, dtype=torch.float32)
            sin_init_(tail, cfg.hidden_dim, index_offset=used)
            flat[used:] = tail
        return flat

    def _metadata(self) -> ModelMetadata:
        from ...checkpoint.formats import config_metadata
        meta = config_metadata(self.lm.cfg)
        md = ModelMetadata.new("transformer")
        first = ("hidden_dim", "num_layers", "num_heads", "vocab_size", "max_seq_len")
        for k in first:
            md.with_custom(k, meta[k])
        for k, v in meta.items():
            if k not in first and k != "architecture":
                md.with_custom(k, v)
        return md

    def write_to(self, writer: BinaryIO, progress=None) -> None:
        write_rustllm_stream(writer, self._reference_flat().numpy(), self._metadata(), progress)

    @classmethod
    def read_from(cls, reader: BinaryIO, device: str = "auto", progress=None) -> "TransformerModel":
        from ...checkpoint.formats import config_from_metadata
        _, params, md = read_rustllm_stream(reader, progress)
        cfg = config_from_metadata(dict(md.custom))
        flat = torch.from_numpy(params.astype("float32", copy=True))
        if flat.numel() < reference_buffer_len(cfg) - (cfg.max_seq_len * cfg.hidden_dim
                                                       + (cfg.vocab_size if cfg.use_bias else 0)):
            raise ProcessingError.shape_mismatch(f"[{reference_buffer_len(cfg)}]",
                                                 f"[{flat.numel()}]")
        dev = _default_device(device)
        lm = DecoderLM(cfg, device=dev, init="zeros", training=False,
                       dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32)
        load_named_into_model(lm, from_reference_flat(flat, cfg))
        used = sum(int(torch.Size(s).numel()) for _, s in reference_offsets(cfg).values())
        return cls(_user_config(cfg), lm, tail=flat[used:].clone(), init="file")

    # ---- PersistentModel-style helpers over files
    def save(self, path: str, fmt: Optional[str] = None) -> None:
        from ...checkpoint.formats import save_model
        fmt = fmt or os.path.splitext(path)[1].lstrip(".").lower()
        if fmt == "rustllm":
            with open(path, "wb") as f:
                self.write_to(f)
        else:
            save_model(self.lm, path, fmt)

    @classmethod
    def load(cls, path: str, device: str = "auto") -> "TransformerModel":
        from ...checkpoint.formats import load_model
        if path.endswith(".rustllm"):
            with open(path, "rb") as f:
                return cls.read_from(f, device=device)
        dev = _default_device(device)
        lm, tail = load_model(path, device=dev)
        return cls(_user_config(lm.cfg), lm, tail=tail, init="file")


def _user_config(cfg: DecoderConfig):
    """The reference-shaped config for reference-shaped models, else the extended one."""
    if (cfg.norm, cfg.pos, cfg.activation, cfg.num_experts) == ("layernorm", "sinusoidal", "gelu", 0):
        return Transformer250MConfig(cfg.hidden_dim, cfg.num_layers, cfg.num_heads,
                                     cfg.intermediate_dim, cfg.vocab_size, cfg.max_seq_len,
                                     cfg.dropout, cfg.attention_dropout, cfg.norm_eps,
                                     cfg.use_bias, "gelu")
    return cfg


class TransformerModelBuilder(ModelBuilder):
    def __init__(self, device: str = "auto", init: str = "reference", verbose: bool = False) -> None:
        self.device, self.init, self.verbose = device, init, verbose

    @staticmethod
    def calculate_num_parameters(config: Transformer250MConfig) -> int:
        return config.buffer_parameters()

    def build(self, config: Union[Transformer250MConfig, DecoderConfig]) -> TransformerModel:
        config.validate()
        dcfg = config.to_decoder(dropout=0.0, attention_dropout=0.0) \
            if isinstance(config, Transformer250MConfig) else config
        dcfg.validate()
        dev = _default_device(self.device)
        if self.verbose:
            print(f"Building enhanced transformer model with {reference_buffer_len(dcfg)} parameters")
        lm = DecoderLM(dcfg, device=dev, init=self.init, training=False,
                       dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32)
        if self.verbose:
            print(f"✓ Created {dcfg.num_layers} transformer blocks")
            print(f"✓ Initialized positional encoding for {dcfg.max_seq_len} positions")
        return TransformerModel(config, lm, init=self.init)


class TransformerModelPlugin(ModelBuilderPlugin):
    def id(self) -> str:
        return "transformer_model"

    def version(self) -> Version:
        return Version(0, 1, 0)

    def capabilities(self) -> PluginCapabilities:
        c = PluginCapabilities.standard()
        for f in ("model_building", "transformer", "250M_params"):
            c.with_feature(f)
        return c

    def create_builder(self, device: str = "auto", init: str = "reference") -> TransformerModelBuilder:
        return TransformerModelBuilder(device=device, init=init)
