"""Architectures register themselves on import."""
from . import gpt2  # noqa: F401
