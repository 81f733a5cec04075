"""Position encodings."""
from __future__ import annotations

from ..weights.spec import MATRIX, TensorSpec
from .base import PositionEncoding


class NoPositions(PositionEncoding):
    """No position signal outside the causal mask."""


class LearnedPositions(PositionEncoding):
    """A learned table added to the token embedding: x0[t] = wte[id] + wpe[position]
    (src/models/gpt2/model.rs:428-450).  The table bounds the longest sequence."""
    adds_to_embedding = True

    def __init__(self, n_positions: int, width: int, init_std: float = 0.02):
        self.n_positions, self.width, self.init_std = n_positions, width, init_std

    def specs(self):
        return {"weight": TensorSpec((self.n_positions, self.width), MATRIX, ("normal", self.init_std))}

    def max_positions(self):
        return self.n_positions
