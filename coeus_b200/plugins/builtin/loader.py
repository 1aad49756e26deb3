"""Model loader plugins.  ``BasicLoaderPlugin`` keeps the reference's identity and behaviour
(plugins/loader-basic/src/lib.rs: formats ``txt`` / ``json``, a pass-through dummy model with
1000 parameters, any other extension is ``Unsupported``) and additionally loads real checkpoints:
``rustllm``, ``safetensors`` and ``gguf`` files go through :mod:`coeus_b200.checkpoint`."""
from __future__ import annotations

from typing import Any, List

from ...core.model import ForwardModel
from ...core.plugin import ModelLoaderPlugin, PluginCapabilities
from ...foundation.error import ProcessingError
from ...foundation.types import Version
from ...models.config import BasicModelConfig


class DummyModel(ForwardModel):
    def __init__(self, config: BasicModelConfig) -> None:
        self._config = config

    def config(self) -> BasicModelConfig:
        return self._config

    def name(self) -> str:
        return "DummyModel"

    def forward(self, input: Any) -> Any:
        return input

    def num_parameters(self) -> int:
        return 1000


class BasicLoaderPlugin(ModelLoaderPlugin):
    def id(self) -> str:
        return "basic_loader"

    def version(self) -> Version:
        return Version(0, 1, 0)

    def capabilities(self) -> PluginCapabilities:
        return (PluginCapabilities.standard().with_feature("model_loading")
                .with_feature("formats:txt,json,rustllm,safetensors,gguf"))

    def supported_formats(self) -> List[str]:
        return ["txt", "json", "rustllm", "safetensors", "gguf"]

    def load_model(self, path: str, device: str = "auto") -> Any:
        if path.endswith((".txt", ".json")):
            return DummyModel(BasicModelConfig())
        if path.endswith((".rustllm", ".safetensors", ".gguf")):
            from .model_transformer import TransformerModel
            return TransformerModel.load(path, device=device)
        raise ProcessingError.unsupported(f"Loading file format: {path}")


CheckpointLoaderPlugin = BasicLoaderPlugin
