"""HTTP serving on top of the continuous batcher."""
from .server import ServingLoop, create_app  # noqa: F401
