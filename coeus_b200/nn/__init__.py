"""Autograd-aware layers built on the sm_100a kernels (see :mod:`.functional`)."""
from . import functional
from .modules import (Block, CausalSelfAttention, CrossEntropyLoss, Embedding, LayerNorm, Linear,
                      MLP, RMSNorm, TransformerLM)

__all__ = ["functional", "Block", "CausalSelfAttention", "CrossEntropyLoss", "Embedding",
           "LayerNorm", "Linear", "MLP", "RMSNorm", "TransformerLM"]
