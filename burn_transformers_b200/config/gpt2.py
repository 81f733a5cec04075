"""GPT-2's configuration with the public checkpoint's field names.

Keys, aliases and defaults (GPT-2 small) follow src/models/gpt2.rs:105-171 of the
reference; the order of the checks follows src/models/gpt2.rs:258-318.
"""
from __future__ import annotations

import dataclasses
from typing import ClassVar

from .base import ModelConfig, field

ACTIVATIONS = ("gelu_new", "gelu")  # src/models/gpt2.rs:78-97
USIZE_MAX = (1 << 64) - 1


@dataclasses.dataclass
class Gpt2Config(ModelConfig):
    FAMILY: ClassVar[str] = "gpt2"
    MODEL_TYPES: ClassVar[tuple[str, ...]] = ("gpt2",)

    model_type: str = field("gpt2")
    vocab_size: int = field(50257)
    n_embd: int = field(768, aliases=("hidden_size",))
    n_layer: int = field(12, aliases=("num_hidden_layers",))
    n_head: int = field(12, aliases=("num_attention_heads",))
    n_positions: int = field(1024, aliases=("max_position_embeddings",))
    n_inner: int | None = field(None)
    activation_function: str = field("gelu_new")
    layer_norm_epsilon: float = field(1e-5)
    scale_attn_weights: bool = field(True)
    scale_attn_by_inverse_layer_idx: bool = field(False)
    reorder_and_upcast_attn: bool = field(False)
    add_cross_attention: bool = field(False)
    tie_word_embeddings: bool = field(True)
    causal: bool = field(True)
    initializer_range: float = field(0.02)

    # derived ------------------------------------------------------------------
    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @property
    def intermediate_size(self) -> int:
        """n_inner, or 4 * n_embd when absent (src/models/gpt2/extents.rs:99-105)."""
        return self.n_inner if self.n_inner is not None else 4 * self.n_embd

    @property
    def max_context(self) -> int:
        """Longest sequence: the learned position table has n_positions rows."""
        return self.n_positions

    def score_scale(self, layer: int) -> float:
        """(1/sqrt(head_dim) if scale_attn_weights) / (layer+1 if scale_attn_by_inverse_layer_idx)
        (src/models/gpt2/model.rs:121-133)."""
        scale = self.head_dim ** -0.5 if self.scale_attn_weights else 1.0
        if self.scale_attn_by_inverse_layer_idx:
            scale /= (layer + 1)
        return scale

    def validate(self) -> None:
        self._check_model_type(self.model_type)
        self._check_extents(("vocab_size", "n_embd", "n_layer", "n_head", "n_positions"))
        self._check_layer_count("n_layer")
        if self.n_embd % self.n_head != 0:
            self._fail("n_head", "must divide n_embd")
        self._check_positive_finite("layer_norm_epsilon")
        self._check_positive_finite("initializer_range")
        if self.reorder_and_upcast_attn:
            self._fail("reorder_and_upcast_attn", "the reordered, upcast attention graph is not implemented")
        if self.add_cross_attention:
            self._fail("add_cross_attention", "cross-attention blocks are not implemented")
        if not self.tie_word_embeddings:
            self._fail("tie_word_embeddings", "the readout must be tied to the token embedding")
        if self.activation_function not in ACTIVATIONS:
            self._fail("activation_function", f"expected one of {list(ACTIVATIONS)}, found `{self.activation_function}`")
        if self.n_inner is not None and self.n_inner <= 0:
            self._fail("n_inner", "must be positive and fit usize")
        for width in (self.vocab_size, self.n_positions, self.intermediate_size, 3):
            if self.n_embd * width > USIZE_MAX:
                self._fail("n_embd", "parameter dimensions overflow usize")
