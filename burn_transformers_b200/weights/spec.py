"""What a model asks of a weight file: tensor names, shapes, and how each is kept."""
from __future__ import annotations

import dataclasses

MATRIX = "matrix"   # operand of a matrix product or an embedding table: kept in the compute dtype
VECTOR = "vector"   # gains, shifts, biases: always 32-bit (a tensor stored in 32-bit stays so)
TABLE = "table"     # integer tables: int32


@dataclasses.dataclass(frozen=True)
class TensorSpec:
    shape: tuple[int, ...]
    kind: str = MATRIX
    # how the random-weights mode fills it: ("normal", std) | ("zeros",) | ("ones",)
    init: tuple = ("zeros",)


@dataclasses.dataclass
class WeightPlan:
    """The tensors of one model, by checkpoint name.

    `namespaces` are prefixes a checkpoint may put before every name; exactly one must
    match, decided by `probe` (src/models/gpt2/checkpoint.rs:46-71 of the reference).
    `ignored` are names (after the prefix) that may be present and are not read.
    `tied` maps an alias that may be physically present to the tensor whose bytes it must equal.
    """
    tensors: dict[str, TensorSpec]
    namespaces: tuple[str, ...] = ("",)
    probe: str | None = None
    ignored: frozenset[str] = frozenset()
    tied: dict[str, str] = dataclasses.field(default_factory=dict)
