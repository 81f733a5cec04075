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


# ---- how a model's tensor is made from the tensors a checkpoint stores ---------------------------------------
# The reference's load plan has the same small vocabulary: Map, Split, Concatenate, Alias
# (src/checkpoint/mapping.rs:139-160, 244-270 of NoahIsCool/burn-transformers).  A model names its tensors as it
# wants them ("[in, out]", queries | keys | values side by side); a source says where each comes from.

@dataclasses.dataclass(frozen=True)
class Stored:
    """A checkpoint tensor taken whole; `transposed`: it is stored with its two axes the other way round."""
    name: str
    transposed: bool = False


@dataclasses.dataclass(frozen=True)
class Split:
    """Piece `index` of a checkpoint tensor cut along `axis` into `sizes` (axis and sizes in the model's orientation,
    that is, after `transposed` has been undone)."""
    name: str
    axis: int
    sizes: tuple[int, ...]
    index: int
    transposed: bool = False


@dataclasses.dataclass(frozen=True)
class Concat:
    """Sources laid side by side along `axis`; `sizes` are their extents along it (None: equal shares)."""
    parts: tuple
    axis: int
    sizes: tuple[int, ...] | None = None


def _flip(shape: tuple[int, ...], transposed: bool) -> tuple[int, ...]:
    if not transposed:
        return tuple(shape)
    if len(shape) != 2:
        raise ValueError(f"only a matrix can be stored transposed, not a tensor of shape {list(shape)}")
    return (shape[1], shape[0])


def stored_shapes(source, shape: tuple[int, ...]) -> list[tuple[str, tuple[int, ...]]]:
    """The checkpoint tensors `source` reads and the shape each must have, given the shape of what it makes."""
    shape = tuple(shape)
    if isinstance(source, Stored):
        return [(source.name, _flip(shape, source.transposed))]
    if isinstance(source, Split):
        if not 0 <= source.index < len(source.sizes) or shape[source.axis] != source.sizes[source.index]:
            raise ValueError(f"piece {source.index} of `{source.name}` cut into {list(source.sizes)} along axis "
                             f"{source.axis} cannot make a tensor of shape {list(shape)}")
        whole = list(shape)
        whole[source.axis] = sum(source.sizes)
        return [(source.name, _flip(tuple(whole), source.transposed))]
    if isinstance(source, Concat):
        n = len(source.parts)
        sizes = source.sizes or ((shape[source.axis] // n,) * n if n and shape[source.axis] % n == 0 else None)
        if sizes is None or len(sizes) != n or sum(sizes) != shape[source.axis]:
            raise ValueError(f"{n} parts of sizes {source.sizes} along axis {source.axis} cannot make a tensor of shape "
                             f"{list(shape)}")
        found = []
        for part, size in zip(source.parts, sizes):
            piece = list(shape)
            piece[source.axis] = size
            found += stored_shapes(part, tuple(piece))
        return found
    raise TypeError(f"not a weight source: {source!r}")


def resolve(source, stored: dict):
    """The tensor `source` describes, from the checkpoint's tensors (torch tensors by name)."""
    import torch
    if isinstance(source, Stored):
        t = stored[source.name]
        return t.t() if source.transposed else t
    if isinstance(source, Split):
        t = stored[source.name]
        t = t.t() if source.transposed else t
        start = sum(source.sizes[:source.index])
        return t.narrow(source.axis, start, source.sizes[source.index])
    if isinstance(source, Concat):
        return torch.cat([resolve(part, stored) for part in source.parts], dim=source.axis)
    raise TypeError(f"not a weight source: {source!r}")


@dataclasses.dataclass
class WeightPlan:
    """The tensors of one model, by checkpoint name.

    `namespaces` are prefixes a checkpoint may put before every name; exactly one must
    match, decided by `probe` (src/models/gpt2/checkpoint.rs:46-71 of the reference).
    `ignored` are names (after the prefix) that may be present and are not read.
    `tied` maps an alias that may be physically present to the tensor whose bytes it must equal.
    `sources` says, for the tensors that are not simply stored under their own name and as they are used, how they
    are made from stored tensors (Stored / Split / Concat); every other tensor is `Stored(its name)`.
    """
    tensors: dict[str, TensorSpec]
    namespaces: tuple[str, ...] = ("",)
    probe: str | None = None
    ignored: frozenset[str] = frozenset()
    tied: dict[str, str] = dataclasses.field(default_factory=dict)
    sources: dict = dataclasses.field(default_factory=dict)

    def source_of(self, name: str):
        return self.sources.get(name) or Stored(name)

    def stored(self) -> dict[str, TensorSpec]:
        """What the checkpoint must hold: stored name -> shape, kind and (for the random-weights mode) init of the
        model tensor it serves.  Two model tensors may read the same stored tensor if they agree on its shape."""
        found: dict[str, TensorSpec] = {}
        for name, spec in self.tensors.items():
            for stored_name, shape in stored_shapes(self.source_of(name), spec.shape):
                seen = found.get(stored_name)
                if seen is not None and (seen.shape != shape or seen.kind != spec.kind):
                    raise ValueError(f"`{stored_name}` is asked for as {list(seen.shape)} {seen.kind} and as "
                                     f"{list(shape)} {spec.kind}")
                found[stored_name] = TensorSpec(shape, spec.kind, spec.init)
        return found
