"""OpenAI-style HTTP front-end for the inference engine (server + request batching)."""
from .server import GenerationService, create_app  # noqa: F401
