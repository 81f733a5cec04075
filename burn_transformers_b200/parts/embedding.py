"""Token embedding and the readout."""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.spec import MATRIX, TensorSpec
from .base import Part
from .linear import linear


class TokenEmbedding(Part):
    """x0[t] = table[id[t]] (+ the position table's row when the position encoding is a learned one)."""

    def __init__(self, vocab: int, width: int, init_std: float = 0.02):
        self.vocab, self.width, self.init_std = vocab, width, init_std

    def specs(self):
        return {"weight": TensorSpec((self.vocab, self.width), MATRIX, ("normal", self.init_std))}

    def forward(self, ctx, positions_part, out32):
        table = positions_part.t_weight if getattr(positions_part, "adds_to_embedding", False) else None
        program = getattr(ctx, "program", None)
        if program is not None:
            program.add_embed(ctx.tokens, ctx.positions if table is not None else None, self.t_weight, table, out32)
            return
        kernels.embed(ctx.tokens, ctx.positions, self.t_weight, table, out32, status=None)


class TiedReadout(Part):
    """logits = h @ table^T with the token embedding's table, no bias, 32-bit logits
    (src/models/gpt2/model.rs:496-513).  Owns no tensor: it borrows the embedding's."""

    accepts_lazy_norm = True

    def __init__(self, embedding: TokenEmbedding):
        self.embedding = embedding

    def forward(self, ctx, h, n_rows: int):
        logits = ctx.ws.take((n_rows, self.embedding.vocab), torch.float32)
        linear(ctx, h, self.embedding.t_weight, None, logits, m=n_rows, w_is_nk=True)
        return logits
