"""Interfaces of the parts a model is put together from.

A part owns its sizes and constants as constructor arguments and its tensors by local names; it
does not know which model it is in.  The model plan maps checkpoint names to (part, local name).

    Norm            forward(ctx, x32, out_dtype, rows=None, n_rows=None) -> normalised rows
    PositionEncoding  `table` to add to the token embedding, and/or rotate(ctx, proj, ...) inside a mixer
    Mixer           cache_need() -> CacheNeed;  forward(ctx, x, residual, entry, owns_cache) adds its
                    output to the 32-bit residual stream in place
    FeedForward     forward(ctx, x, residual) adds its output to the residual stream in place
    Block           forward(ctx, residual, entry, owns_cache) arranges norms, mixer and feed-forward

`x` holds the step's tokens as rows, packed sequence after sequence (no padding); `ctx`
(engine.step.StepContext) says which row belongs to which sequence and position.
"""
from __future__ import annotations

import torch

from ..cache.spec import CacheNeed
from ..weights.spec import TensorSpec


class Part:
    """Something with tensors of its own."""

    def specs(self) -> dict[str, TensorSpec]:
        return {}

    # Names of [in, out] matrices that are only ever the right-hand side of parts.linear.linear.  In bfloat16
    # they are kept transposed, [out, in] with the input axis contiguous: the layout the tensor-core and the
    # weight-streaming kernels read (both operands K-major).  `nk_<name>` says which layout `t_<name>` has.
    linear_weights: tuple[str, ...] = ()

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        for name in self.specs():
            tensor = tensors[name]
            attr = name.replace(".", "_")
            if name in self.linear_weights:
                transposed = tensor.dtype == torch.bfloat16
                if transposed:
                    tensor = tensor.t().contiguous()
                setattr(self, "nk_" + attr, transposed)
            setattr(self, "t_" + attr, tensor)

    # Parts made only of this library's kernels can be captured in a CUDA graph.
    graph_safe = True


class Norm(Part):
    # A norm that the weight-streaming products can apply to their rows on the way in (LayerNorm semantics: tensors
    # `t_weight`, `t_bias` if `has_bias`, `eps`) sets `fusable`.  `fused_kind` names what the fused decode step may do
    # in its place: "layernorm" or "rmsnorm" (rows scaled by the root of their mean square plus `eps`, times `t_weight`,
    # plus `t_bias` if `has_bias`); None: the norm runs as its own kernels and the step as separate kernels.
    fusable = False
    fused_kind: str | None = None

    def forward(self, ctx, x32, out_dtype, rows=None, n_rows=None, lazy=False):
        """`lazy` allows (never obliges) the norm to return a handle that the consumer's first matrix product
        resolves inside its kernel; only consumers that set `accepts_lazy_norm` are given one."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Learned tables add to the embedding; rotary kinds act on queries and keys inside a mixer."""
    adds_to_embedding = False
    rotates = False

    def max_positions(self) -> int | None:
        return None

    def rotate(self, ctx, proj, n_heads: int, n_kv_heads: int, head_dim: int) -> None:
        """For a kind with `rotates`: turns the query and key channels of the step's projections `proj`
        ([tokens, (n_heads + 2 * n_kv_heads) * head_dim]: queries, keys, values) in place, each token by its own
        position `ctx.positions`, angles in 32-bit.  A mixer calls this before it files the keys."""
        raise NotImplementedError


class Mixer(Part):
    accepts_lazy_norm = False   # True: `x` is only ever handed to parts.linear.linear

    def cache_need(self) -> CacheNeed:
        return CacheNeed()

    def forward(self, ctx, x, residual, entry: int, owns_cache: bool = True) -> None:
        raise NotImplementedError


class FeedForward(Part):
    accepts_lazy_norm = False

    def forward(self, ctx, x, residual) -> None:
        raise NotImplementedError


class Block(Part):
    def parts(self) -> dict[str, Part]:
        raise NotImplementedError

    def cache_need(self) -> CacheNeed:
        raise NotImplementedError

    def forward(self, ctx, residual, entry: int, owns_cache: bool = True) -> None:
        raise NotImplementedError
