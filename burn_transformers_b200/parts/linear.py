"""Matrix products of the parts: picks the kernel for the element type and the shape."""
from __future__ import annotations

import torch

from .. import kernels


class LazyNorm:
    """Rows that are still to be normalised: (32-bit rows, the norm part, an optional row index).

    A product that can normalise on the way in takes it as it is; anything else calls `materialize`."""

    def __init__(self, norm, x32, rows, n_rows):
        self.norm, self.x32, self.rows, self.n_rows = norm, x32, rows, n_rows
        self.dtype = torch.bfloat16

    def materialize(self, ctx):
        return self.norm.apply(ctx, self.x32, torch.bfloat16, self.rows, self.n_rows)


def linear(ctx, a, w, bias, out, *, m, w_is_nk=False, activation=None, residual=None):
    """out[:m] = act(a[:m] @ w + bias) (+ residual[:m]);  w is [K, N], or [N, K] when `w_is_nk`.

    32-bit operands always take the plain fused-multiply-add kernel: the 32-bit path has no reduced-precision
    matrix mode.  bfloat16 products of at most 16 rows take a weight-streaming kernel, which can also normalise
    its rows on the way in; 17 to 64 rows ([N, K] weights) take the kernel that is fed by tensor-map copies (large
    weights with a short K the tcgen05 product for many rows); up to 128 rows over a large weight (any K at up to 16
    rows, a long K above) take the tcgen05 product with the weights on the M side; with more rows they run on the
    tcgen05 tensor cores."""
    program = getattr(ctx, "program", None)
    if program is not None:      # a fused decode step is being recorded: this product becomes one of its phases
        program.add_linear(a, w, bias, out, m=m, w_is_nk=w_is_nk, activation=activation, residual=residual)
        return
    lazy = isinstance(a, LazyNorm)
    n = w.shape[0] if w_is_nk else w.shape[1]
    k = w.shape[1] if w_is_nk else w.shape[0]
    if (w.dtype == torch.bfloat16 and w_is_nk and n < 8192 and kernels.linear_few_tcgen05_supports(m, n, k)
            and ((m <= 16 and n * k >= 7_000_000) or (16 < m <= 64 and k >= 4096 and n * k >= 6_000_000)
                 or (64 < m <= 128 and k >= 4096 and n * k >= 3_000_000))):
        # a large weight: the tcgen05 product with the weights on the tensor cores' M side and K cut over a cluster.
        # Measured in a graph with weights that rotate through more than L2 holds, against the kernel that would take
        # the shape otherwise: 64 rows, 1600 x 6400: 15.4 against 21.9 us; 128 rows: 21.0 against 32.5 us, 1024 x 4096:
        # 17.9 against 22.1; 8 rows, 4800 x 1600: 9.5 against 11.6 us, 6400 x 1600: 10.4 against 12.6, and the decode step
        # of GPT-2 XL outside the fused step at 16 rows 3.36 against 4.94 ms (below 7 M weights the kernels for few
        # rows win: 5120 x 1280 at 8 rows 6.9 against 8.8 us)
        if lazy:
            a = a.materialize(ctx)
        kernels.linear_few_tcgen05(a, w, bias, out, m=m, activation=activation, residual=residual)
        return
    if (w.dtype == torch.bfloat16 and w_is_nk and 16 < m <= 64 and n * k >= 6_000_000 and k <= 2048 and n < 8192
            and kernels.linear_tcgen05_supports(m, n, k)):
        # a large weight with a short K: the tcgen05 product streams it faster even with half of its 128 rows empty
        # (measured at 64 rows: 4800 x 1600 in 10.3 us against 17.2 us, 6400 x 1600 in 10.7 against 17.6; a long K
        # (1600 x 6400: 31.8 against 22.3 us), small weights (2304 x 768: 6.2 against 5.1 us) and a readout, for which
        # the kernel below has blocks of 64 columns, stay there)
        if lazy:
            a = a.materialize(ctx)
        kernels.linear_tcgen05(a, w, bias, out, m=m, activation=activation, residual=residual)
        return
    if w.dtype == torch.bfloat16 and w_is_nk and 16 < m <= 64 and kernels.linear_mid_supports(m, n, k):
        # more than one 16-row tile: all rows of a block of 16 columns in one block, fed by tensor-map copies
        # (the weight-streaming kernels below spend an instruction stream per 16 rows)
        if lazy:
            a = a.materialize(ctx)
        kernels.linear_mid(a, w, bias, out, m=m, activation=activation, residual=residual)
        return
    if w.dtype == torch.bfloat16 and m <= 64:
        fuse = lazy and m <= 16 and a.norm.fusable
        if w_is_nk and n >= 8192 and kernels.linear_stream_supports(m, n, k, fuse):
            # a wide [N, K] table (the readout): long weight rows, streamed straight into registers
            if lazy and not fuse:
                a, lazy = a.materialize(ctx), False
            norm = (a.x32, a.norm.t_weight, a.norm.t_bias if a.norm.has_bias else None, a.norm.eps, a.rows) if lazy else None
            kernels.linear_stream(None if lazy else a, w, bias, out, m=m, activation=activation, residual=residual,
                                  norm=norm)
            return
        if kernels.linear_skinny_supports(m, n, k, w_is_nk, fuse):
            if lazy and not fuse:
                a, lazy = a.materialize(ctx), False
            norm = (a.x32, a.norm.t_weight, a.norm.t_bias if a.norm.has_bias else None, a.norm.eps, a.rows) if lazy else None
            kernels.linear_skinny(None if lazy else a, w, bias, out, m=m, w_is_nk=w_is_nk, activation=activation,
                                  residual=residual, norm=norm)
            return
    if lazy:
        a = a.materialize(ctx)
    if w.dtype == torch.bfloat16 and w_is_nk and m > 64 and kernels.linear_tcgen05_supports(m, n, k):
        kernels.linear_tcgen05(a, w, bias, out, m=m, activation=activation, residual=residual)
        return
    kernels.linear_simt(a, w, bias, out, m=m, w_is_nk=w_is_nk, activation=activation, residual=residual)
