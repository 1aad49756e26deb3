"""Model contracts (counterpart of src/core/model.rs): the ``Model`` / ``ForwardModel`` /
``TrainableModel`` / ``GenerativeModel`` / ``BatchedModel`` / ``ModelBuilder`` /
``PersistentModel`` / ``QuantizableModel`` interfaces, ``Tensor`` (shape-checked; data is a
``torch.Tensor`` here instead of a ``Vec<f32>``), ``Layer`` / ``Attention``, the optimizer, loss,
noise-schedule and sampler interfaces, generation configs, and the typed configurations (kept in
:mod:`coeus_b200.models.config`)."""
from __future__ import annotations

import abc
from dataclasses import dataclass
from typing import Any, List, Optional, Sequence

import torch

from ..foundation.error import ProcessingError
from ..foundation.types import Shape
from ..models.config import BasicModelConfig, DecoderConfig, Transformer250MConfig  # noqa: F401


class ModelConfig(abc.ABC):
    @abc.abstractmethod
    def model_dim(self) -> int: ...

    @abc.abstractmethod
    def head_count(self) -> int: ...

    @abc.abstractmethod
    def layer_count(self) -> int: ...

    def validate(self) -> None:
        return None


ModelConfig.register(Transformer250MConfig)


class VocabularyConfig(abc.ABC):
    @abc.abstractmethod
    def vocab_size(self) -> int: ...

    def pad_token_id(self) -> Optional[int]:
        return None


class SequenceConfig(abc.ABC):
    @abc.abstractmethod
    def max_seq_len(self) -> int: ...

    def use_positional_encoding(self) -> bool:
        return True


class DropoutConfig(abc.ABC):
    @abc.abstractmethod
    def dropout(self) -> float: ...

    def attention_dropout(self) -> Optional[float]:
        return None


class Model(abc.ABC):
    @abc.abstractmethod
    def config(self) -> Any: ...

    @abc.abstractmethod
    def name(self) -> str: ...


class ForwardModel(Model):
    @abc.abstractmethod
    def forward(self, input: Any) -> Any: ...

    @abc.abstractmethod
    def num_parameters(self) -> int: ...


class TrainableModel(Model):
    @abc.abstractmethod
    def train_step(self, input: Any, optimizer_state: Any) -> Any: ...

    @abc.abstractmethod
    def update_parameters(self, gradients: Any) -> None: ...

    @abc.abstractmethod
    def compute_loss(self, data: Any) -> float: ...

    @abc.abstractmethod
    def is_training(self) -> bool: ...

    @abc.abstractmethod
    def set_training(self, training: bool) -> None: ...


class GenerativeModel(ForwardModel):
    @abc.abstractmethod
    def generate(self, input: Any, config: Any) -> List[int]: ...


class BatchedModel(Model):
    @abc.abstractmethod
    def forward_batch(self, batch: Any) -> Any: ...


class ModelBuilder(abc.ABC):
    @abc.abstractmethod
    def build(self, config: Any) -> Model: ...

    def validate_config(self, config: Any) -> None:
        config.validate()


class PersistentModel(Model):
    @abc.abstractmethod
    def save(self) -> bytes: ...

    @classmethod
    @abc.abstractmethod
    def load(cls, data: bytes) -> "PersistentModel": ...


class QuantizableModel(Model):
    @abc.abstractmethod
    def quantize(self, config: Any) -> None: ...

    @abc.abstractmethod
    def is_quantized(self) -> bool: ...


class Tensor:
    """``Tensor{shape, data}`` (model.rs:203-249): ``new`` checks ``shape.numel() == len(data)``
    and raises ``ShapeMismatch`` otherwise."""

    def __init__(self, shape: Shape, data: Any) -> None:
        t = data if isinstance(data, torch.Tensor) else torch.tensor(list(data), dtype=torch.float32)
        if shape.numel() != t.numel():
            raise ProcessingError.shape_mismatch(f"numel={shape.numel()}", f"len={t.numel()}")
        self.shape = shape
        self.data = t.reshape(-1)

    new = classmethod(lambda cls, shape, data: cls(shape, data))

    @classmethod
    def zeros(cls, shape: Shape) -> "Tensor":
        return cls(shape, torch.zeros(shape.numel()))

    @classmethod
    def ones(cls, shape: Shape) -> "Tensor":
        return cls(shape, torch.ones(shape.numel()))

    def as_slice(self) -> torch.Tensor:
        return self.data

    as_mut_slice = as_slice

    def view(self) -> torch.Tensor:
        return self.data.view(*self.shape.dims())


class Layer(abc.ABC):
    @abc.abstractmethod
    def forward(self, input: Any) -> Any: ...

    @abc.abstractmethod
    def num_parameters(self) -> int: ...


class Attention(Layer):
    @abc.abstractmethod
    def attend(self, query: Tensor, key: Tensor, value: Tensor,
               mask: Optional[Tensor] = None) -> Tensor: ...


class OptimizerState(abc.ABC):
    @abc.abstractmethod
    def reset(self) -> None: ...

    @abc.abstractmethod
    def learning_rate(self) -> float: ...

    @abc.abstractmethod
    def set_learning_rate(self, lr: float) -> None: ...

    @abc.abstractmethod
    def step_count(self) -> int: ...

    @abc.abstractmethod
    def increment_step(self) -> None: ...


class Loss(abc.ABC):
    @abc.abstractmethod
    def compute(self, predictions: Sequence[float], targets: Sequence[float]) -> float: ...

    @abc.abstractmethod
    def gradient(self, predictions: Sequence[float], targets: Sequence[float]) -> List[float]: ...


class MSELoss(Loss):
    """The loss of the reference's training example (examples/training_example.rs:64-103)."""

    def compute(self, predictions, targets) -> float:
        if len(predictions) != len(targets):
            raise ProcessingError.shape_mismatch(str(len(targets)), str(len(predictions)))
        return sum((p - t) ** 2 for p, t in zip(predictions, targets)) / max(1, len(predictions))

    def gradient(self, predictions, targets) -> List[float]:
        n = max(1, len(predictions))
        return [2.0 * (p - t) / n for p, t in zip(predictions, targets)]


class NoiseSchedule(abc.ABC):
    @abc.abstractmethod
    def num_steps(self) -> int: ...

    @abc.abstractmethod
    def beta(self, timestep: int) -> float: ...

    @abc.abstractmethod
    def alpha_bar(self, timestep: int) -> float: ...


class DiffusionSampler(abc.ABC):
    @abc.abstractmethod
    def sample_step(self, current, predicted_noise, timestep: int,
                    noise_schedule: NoiseSchedule): ...

    @abc.abstractmethod
    def is_deterministic(self) -> bool: ...


class GenerationConfig(abc.ABC):
    @abc.abstractmethod
    def max_length(self) -> int: ...

    @abc.abstractmethod
    def temperature(self) -> float: ...


@dataclass
class BasicGenerationConfig:
    """model.rs:719-753 (defaults 100 / 1.0 / None / None)."""

    max_length: int = 100
    temperature: float = 1.0
    top_k: Optional[int] = None
    top_p: Optional[float] = None


GenerationConfig.register(BasicGenerationConfig)
