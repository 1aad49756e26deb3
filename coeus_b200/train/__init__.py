"""Training engine."""
from .trainer import TrainConfig, Trainer  # noqa: F401
