"""Inference: paged KV cache, sampling, and the generation engine."""
from .engine import InferenceEngine  # noqa: F401
from .kv_cache import PagedKVCache  # noqa: F401
