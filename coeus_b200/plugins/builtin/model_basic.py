"""Basic model plugin (plugins/model-basic/src/lib.rs): ``forward`` is the identity and
``num_parameters = V*D + L*D^2*4 + L*D^2*8``."""
from __future__ import annotations

from typing import Any

from ...core.model import ForwardModel, ModelBuilder
from ...core.plugin import ModelBuilderPlugin, PluginCapabilities
from ...foundation.types import Version
from ...models.config import BasicModelConfig


class BasicModel(ForwardModel):
    def __init__(self, config: BasicModelConfig) -> None:
        self._config = config

    def config(self) -> BasicModelConfig:
        return self._config

    def name(self) -> str:
        return "BasicModel"

    def forward(self, input: Any) -> Any:
        return input

    def num_parameters(self) -> int:
        c = self._config
        return (c.vocab_size * c.model_dim + c.layer_count * c.model_dim * c.model_dim * 4
                + c.layer_count * c.model_dim * c.model_dim * 8)


class BasicModelBuilder(ModelBuilder):
    new = classmethod(lambda cls: cls())

    def build(self, config: BasicModelConfig) -> BasicModel:
        config.validate()
        return BasicModel(config)


class BasicModelPlugin(ModelBuilderPlugin):
    def id(self) -> str:
        return "basic_model"

    def version(self) -> Version:
        return Version(0, 1, 0)

    def capabilities(self) -> PluginCapabilities:
        return PluginCapabilities.standard().with_feature("model_building")

    def create_builder(self) -> BasicModelBuilder:
        return BasicModelBuilder()
