"""Matrix products of the parts: picks the kernel for the element type and the shape."""
from __future__ import annotations

import torch

from .. import kernels


def linear(ctx, a, w, bias, out, *, m, w_is_nk=False, activation=None, residual=None):
    """out[:m] = act(a[:m] @ w + bias) (+ residual[:m]).

    32-bit operands always take the plain fused-multiply-add kernel: the 32-bit path has no
    reduced-precision matrix mode.
    """
    kernels.linear_simt(a, w, bias, out, m=m, w_is_nk=w_is_nk, activation=activation, residual=residual)
