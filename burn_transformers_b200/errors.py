"""Error types of the library, one per stage, so a caller can tell where a request failed.

The classes follow the reference's single error enum (src/error.rs:13-190 of
NoahIsCool/burn-transformers): Configuration{field, reason}, Shape, Cache,
Checkpoint*, Generation, UnsupportedArchitecture, BackendCapability.
"""
from __future__ import annotations


class BurnTransformersError(Exception):
    """Base class of every error this library raises on purpose."""


class ConfigError(BurnTransformersError):
    """A configuration field is missing, has the wrong type or breaks an invariant.

    Printed as `architecture.field: reason` (src/models/config.rs:70-80).
    """

    def __init__(self, architecture: str, field: str, reason: str):
        self.architecture, self.field, self.reason = architecture, field, reason
        super().__init__(f"{architecture}.{field}: {reason}")


class UnsupportedArchitecture(BurnTransformersError):
    """config.json names a model_type that no registered architecture executes."""


class CheckpointError(BurnTransformersError):
    """The weight file cannot be read, or its tensors do not match the model.

    `missing`, `unexpected` and `mismatched` hold everything that was wrong, so
    one failed load tells the whole story.
    """

    def __init__(self, message: str, *, missing=(), unexpected=(), mismatched=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.mismatched = list(mismatched)
        super().__init__(message)


class ShapeError(BurnTransformersError):
    """A tensor or a list handed to the library has the wrong extent or dtype."""


class CacheError(BurnTransformersError):
    """The cache cannot take a request: no slot, no page, capacity exceeded, a slot misused."""


class GenerationError(BurnTransformersError):
    """A generation option is invalid, or generation met a non-finite score."""


class KernelError(BurnTransformersError):
    """The compiled CUDA library is missing, failed to build, or refused a size."""
