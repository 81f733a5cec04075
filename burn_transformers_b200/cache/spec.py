"""What a layer asks of the cache."""
from __future__ import annotations

import dataclasses

import torch

PAGE_SIZE = 64  # tokens per page; the kernels' page_size


@dataclasses.dataclass(frozen=True)
class KvSpec:
    """Keys and values per position: all of them (`window` None) or the last `window`."""
    n_kv_heads: int
    head_dim: int
    window: int | None = None

    def __post_init__(self):
        if self.n_kv_heads <= 0 or self.head_dim <= 0:
            raise ValueError("KvSpec: heads and head_dim must be positive")
        if self.window is not None and self.window <= 0:
            raise ValueError("KvSpec: window must be positive")


@dataclasses.dataclass(frozen=True)
class StateSpec:
    """A tensor of fixed size per sequence (for instance a recurrent state), zero for a new sequence."""
    name: str
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclasses.dataclass(frozen=True)
class CacheNeed:
    """The cache needs of one layer call: time-indexed keys/values and/or fixed-size states."""
    kv: KvSpec | None = None
    states: tuple[StateSpec, ...] = ()


@dataclasses.dataclass(frozen=True)
class CacheConfig:
    """Geometry of a cache (the reference's CacheConfig{sequence_count, capacity}, src/cache/config.rs:30-85,
    restated for pages): `max_tokens` is the most tokens live sequences hold at any time, each sequence's
    count rounded up to a whole page; `max_slots` the most live sequences; `max_context` the longest
    sequence."""
    max_tokens: int
    max_slots: int
    max_context: int

    def __post_init__(self):
        for name in ("max_tokens", "max_slots", "max_context"):
            if getattr(self, name) <= 0:
                from ..errors import CacheError
                raise CacheError(f"cache.{name} must be greater than zero")
