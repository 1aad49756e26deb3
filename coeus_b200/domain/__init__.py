"""Domain layer (counterpart of src/domain/): value objects, aggregates, events, repository
interfaces and services per bounded context."""
from . import inference, modeling, persistence, tokenization, training  # noqa: F401
