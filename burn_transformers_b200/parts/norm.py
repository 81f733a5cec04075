"""Normalisation parts."""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.spec import VECTOR, TensorSpec
from .base import Norm
from .linear import LazyNorm


class LayerNorm(Norm):
    """Affine LayerNorm over the last axis, biased variance, statistics in 32-bit
    (src/models/gpt2/model.rs:143-148, 235-239 of the reference)."""

    def __init__(self, width: int, eps: float, bias: bool = True):
        self.width, self.eps, self.has_bias = width, float(eps), bias

    def specs(self):
        specs = {"weight": TensorSpec((self.width,), VECTOR, ("ones",))}
        if self.has_bias:
            specs["bias"] = TensorSpec((self.width,), VECTOR, ("zeros",))
        return specs

    fusable = True      # linear kernels know how to apply this norm to their rows on the way in
    fused_kind = "layernorm"

    def forward(self, ctx, x32, out_dtype, rows=None, n_rows=None, lazy=False):
        """Normalised rows; with `lazy` (and bfloat16 output, few rows) a handle that the next matrix product
        resolves, normalising inside its own kernel."""
        n = n_rows if n_rows is not None else ctx.n_tokens
        if lazy and out_dtype == torch.bfloat16 and n <= 16:
            return LazyNorm(self, x32, rows, n)
        return self.apply(ctx, x32, out_dtype, rows, n)

    def apply(self, ctx, x32, out_dtype, rows, n):
        out = ctx.ws.take((n, self.width), out_dtype)
        kernels.layernorm(x32, self.t_weight, self.t_bias if self.has_bias else None, out, self.eps, rows=rows, n_rows=n)
        return out
