"""Feed-forward parts."""
from __future__ import annotations

from ..weights.spec import MATRIX, VECTOR, TensorSpec
from .base import FeedForward
from .linear import linear

ACTIVATIONS = ("gelu_new", "gelu")


class DenseFeedForward(FeedForward):
    """down(act(up(x))), added to the residual stream (src/feed_forward.rs:111-114 of the reference).
    `gelu_new` is the tanh form, `gelu` the erf form; both are evaluated in 32-bit on the
    accumulator and rounded once."""

    accepts_lazy_norm = True
    linear_weights = ("up.weight", "down.weight")

    def __init__(self, width: int, inner: int, activation: str, *, bias: bool = True, init_std: float = 0.02,
                 down_init_std: float | None = None):
        if activation not in ACTIVATIONS:
            raise ValueError(f"activation must be one of {ACTIVATIONS}, found {activation!r}")
        self.width, self.inner, self.activation, self.has_bias = width, inner, activation, bias
        self.init_std = init_std
        self.down_init_std = init_std if down_init_std is None else down_init_std

    def specs(self):
        specs = {"up.weight": TensorSpec((self.width, self.inner), MATRIX, ("normal", self.init_std)),
                 "down.weight": TensorSpec((self.inner, self.width), MATRIX, ("normal", self.down_init_std))}
        if self.has_bias:
            specs["up.bias"] = TensorSpec((self.inner,), VECTOR, ("zeros",))
            specs["down.bias"] = TensorSpec((self.width,), VECTOR, ("zeros",))
        return specs

    def forward(self, ctx, x, residual):
        n = ctx.n_tokens
        hidden = ctx.ws.take((n, self.inner), ctx.dtype)
        linear(ctx, x, self.t_up_weight, self.t_up_bias if self.has_bias else None, hidden, m=n,
               activation=self.activation, w_is_nk=self.nk_up_weight)
        linear(ctx, hidden, self.t_down_weight, self.t_down_bias if self.has_bias else None, residual, m=n,
               residual=residual, w_is_nk=self.nk_down_weight)
