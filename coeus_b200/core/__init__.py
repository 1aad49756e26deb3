"""Core API layer: traits, plugin / tokenizer / model contracts, configuration store and the
``.rustllm`` serialization (counterpart of ``src/core/`` in the reference)."""
