"""GPT-2 as a plan of parts: pre-LayerNorm blocks with fused-QKV causal attention and a GELU
feed-forward, a learned position table, and a readout tied to the token embedding.

Checkpoint names and layouts follow src/models/gpt2/checkpoint.rs:103-189 of the reference
(NoahIsCool/burn-transformers); Conv1D weights are [in, out] and are used as stored
(src/models/gpt2/model.rs:136-137).  The reference splits c_attn into three matrices at load;
here it stays one fused projection, which is the same arithmetic.
"""
from __future__ import annotations

import math

from ..config.gpt2 import Gpt2Config
from ..config.registry import Architecture, register_architecture
from ..errors import ConfigError
from ..engine.model import LayerCall, ModelPlan
from ..parts import (CausalSelfAttention, DenseFeedForward, LayerNorm, LearnedPositions, PreNormBlock, TiedReadout,
                     TokenEmbedding)


def build_gpt2(config: Gpt2Config) -> ModelPlan:
    config.validate()
    # what the configuration allows but this engine does not run is refused here, by field, before anything is built
    if config.head_dim > CausalSelfAttention.MAX_HEAD_DIM:
        raise ConfigError("gpt2", "n_head", f"n_embd / n_head = {config.head_dim} exceeds the largest head size the "
                                            f"attention kernels take ({CausalSelfAttention.MAX_HEAD_DIM})")
    if not config.causal:
        # (the reference's `causal` is a knob of its stateless forward, src/models/gpt2/model.rs:22-24; with a cache a
        # token never sees later ones, so a non-causal forward cannot be reproduced step by step)
        raise ConfigError("gpt2", "causal", "an engine with a cache decodes causally; `causal: false` is not executable")
    d, std = config.n_embd, config.initializer_range
    # projections that write into the residual stream start narrower (src/models/gpt2.rs:188-222)
    residual_std = std / math.sqrt(2.0 * config.n_layer)
    embedding = TokenEmbedding(config.vocab_size, d, std)
    positions = LearnedPositions(config.n_positions, d, std)
    final_norm = LayerNorm(d, config.layer_norm_epsilon)
    names = {"wte.weight": (embedding, "weight"), "wpe.weight": (positions, "weight"),
             "ln_f.weight": (final_norm, "weight"), "ln_f.bias": (final_norm, "bias")}
    blocks = []
    ignored = set()
    for i in range(config.n_layer):
        norm1 = LayerNorm(d, config.layer_norm_epsilon)
        norm2 = LayerNorm(d, config.layer_norm_epsilon)
        attention = CausalSelfAttention(d, config.n_head, config.n_head, config.head_dim, config.score_scale(i),
                                        causal=config.causal, bias=True, init_std=std, out_init_std=residual_std)
        mlp = DenseFeedForward(d, config.intermediate_size, config.activation_function, bias=True, init_std=std,
                               down_init_std=residual_std)
        blocks.append(PreNormBlock(norm1, attention, norm2, mlp))
        p = f"h.{i}."
        names.update({
            p + "ln_1.weight": (norm1, "weight"), p + "ln_1.bias": (norm1, "bias"),
            p + "attn.c_attn.weight": (attention, "qkv.weight"), p + "attn.c_attn.bias": (attention, "qkv.bias"),
            p + "attn.c_proj.weight": (attention, "out.weight"), p + "attn.c_proj.bias": (attention, "out.bias"),
            p + "ln_2.weight": (norm2, "weight"), p + "ln_2.bias": (norm2, "bias"),
            p + "mlp.c_fc.weight": (mlp, "up.weight"), p + "mlp.c_fc.bias": (mlp, "up.bias"),
            p + "mlp.c_proj.weight": (mlp, "down.weight"), p + "mlp.c_proj.bias": (mlp, "down.bias"),
        })
        # legacy causal-mask buffers some exports carry (src/models/gpt2/checkpoint.rs:169-174)
        ignored.update({p + "attn.bias", p + "attn.masked_bias"})
    return ModelPlan(
        config=config, embedding=embedding, positions=positions, blocks=blocks,
        schedule=[LayerCall(i) for i in range(config.n_layer)], final_norm=final_norm,
        readout=TiedReadout(embedding), names=names, vocab=config.vocab_size, width=d,
        max_context=config.n_positions, namespaces=("", "transformer."), probe="wte.weight",
        ignored=frozenset(ignored), tied={"lm_head.weight": "wte.weight"})


GPT2 = register_architecture(Architecture("gpt2", ("gpt2",), Gpt2Config, build_gpt2), replace=True)
