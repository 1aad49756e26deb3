"""Model family: configs, parameter layouts and the decoder-only transformer."""
from .config import BasicModelConfig, DecoderConfig, Transformer250MConfig  # noqa: F401
