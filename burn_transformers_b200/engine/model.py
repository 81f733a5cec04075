"""A decoder as data: parts, the order in which layers run, and the checkpoint names of their tensors.

Nothing here names an architecture.  An architecture's builder (for instance models/gpt2.py)
returns a ModelPlan; the engine runs any plan.
"""
from __future__ import annotations

import dataclasses

import torch

from ..cache.spec import CacheNeed
from ..config.base import ModelConfig
from ..parts.base import Block, Norm, Part, PositionEncoding
from ..weights.spec import TensorSpec, WeightPlan


@dataclasses.dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: which block runs, and whose cache it uses.

    `cache` None: the call owns a cache entry of its own (so a block named twice keeps separate
    keys and values per call).  `cache` = index of an earlier call: this call reads that call's
    entry and writes nothing.
    """
    block: int
    cache: int | None = None


@dataclasses.dataclass
class ModelPlan:
    config: ModelConfig
    embedding: Part
    positions: PositionEncoding
    blocks: list[Block]
    schedule: list[LayerCall]
    final_norm: Norm
    readout: Part
    names: dict[str, tuple[Part, str]]            # checkpoint name -> (part, local tensor name)
    vocab: int
    width: int
    max_context: int
    namespaces: tuple[str, ...] = ("",)
    probe: str | None = None
    ignored: frozenset[str] = frozenset()
    tied: dict[str, str] = dataclasses.field(default_factory=dict)
    # for a name of `names` whose tensor is not stored under that name and as the part uses it: how it is made from
    # the checkpoint's tensors (weights.spec.Stored / Split / Concat); the name is then only the model's own
    sources: dict = dataclasses.field(default_factory=dict)

    def __post_init__(self):
        for index, call in enumerate(self.schedule):
            if not (0 <= call.block < len(self.blocks)):
                raise ValueError(f"schedule[{index}] names block {call.block} of {len(self.blocks)}")
            if call.cache is not None:
                if not (0 <= call.cache < index) or self.schedule[call.cache].cache is not None:
                    raise ValueError(f"schedule[{index}] must read the cache of an earlier call that owns one")

    @property
    def weights(self) -> WeightPlan:
        tensors: dict[str, TensorSpec] = {}
        for name, (part, local) in self.names.items():
            tensors[name] = part.specs()[local]
        return WeightPlan(tensors, self.namespaces, self.probe, self.ignored, dict(self.tied), dict(self.sources))

    def cache_needs(self) -> list[CacheNeed]:
        """One entry per call of the schedule; readers of another call's cache need nothing."""
        return [self.blocks[c.block].cache_need() if c.cache is None else CacheNeed() for c in self.schedule]

    def cache_entry(self, call_index: int) -> tuple[int, bool]:
        call = self.schedule[call_index]
        return (call_index, True) if call.cache is None else (call.cache, False)

    def all_parts(self) -> list[Part]:
        found: list[Part] = [self.embedding, self.positions, self.final_norm, self.readout]
        for block in self.blocks:
            found.append(block)
            found.extend(block.parts().values())
        return found

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        """Hands every part its tensors under their local names."""
        per_part: dict[int, tuple[Part, dict[str, torch.Tensor]]] = {}
        for name, (part, local) in self.names.items():
            per_part.setdefault(id(part), (part, {}))[1][local] = tensors[name]
        for part, local_tensors in per_part.values():
            part.bind(local_tensors)

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", True) for p in self.all_parts())

    def forward(self, ctx):
        """Runs the step's tokens through every layer call; returns 32-bit logits at the wanted rows."""
        residual = ctx.ws.take((ctx.n_tokens, self.width), torch.float32)
        self.embedding.forward(ctx, self.positions, residual)
        for index, call in enumerate(self.schedule):
            entry, owns = self.cache_entry(index)
            self.blocks[call.block].forward(ctx, residual, entry, owns)
        if getattr(ctx, "side", None) is not None:
            ctx.side.join()       # (what parts ran beside the step must be done before the step's scratch is used again)
        if ctx.n_want == 0:
            return None
        h = self.final_norm.forward(ctx, residual, ctx.dtype, rows=ctx.want_rows, n_rows=ctx.n_want,
                                    lazy=getattr(self.readout, "accepts_lazy_norm", False))
        return self.readout.forward(ctx, h, ctx.n_want)
