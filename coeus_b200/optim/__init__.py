"""Optimizers over the flat parameter buffers."""
from .adamw import AdamW, AdamWConfig  # noqa: F401
from .sgd import SGD  # noqa: F401
