"""Checkpoint formats: ``.rustllm`` (bit-exact with the reference), SafeTensors, GGUF, and sharded
training checkpoints."""
from .formats import (load_gguf, load_model, load_safetensors, save_gguf, save_model,  # noqa: F401
                      save_safetensors)
