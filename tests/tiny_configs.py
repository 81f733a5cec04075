"""Two tiny GPT-2 configurations that differ in every size and option, and helpers to make model folders."""
from __future__ import annotations

import numpy as np

import burn_transformers_b200 as bt

TINY_A = dict(model_type="gpt2", n_layer=2, n_embd=64, n_head=4, n_inner=256, vocab_size=512, n_positions=128,
              layer_norm_epsilon=1e-5, activation_function="gelu_new", scale_attn_weights=True,
              scale_attn_by_inverse_layer_idx=False)
TINY_B = dict(model_type="gpt2", n_layer=3, n_embd=96, n_head=3, n_inner=320, vocab_size=1000, n_positions=256,
              layer_norm_epsilon=1e-6, activation_function="gelu", scale_attn_weights=True,
              scale_attn_by_inverse_layer_idx=True)
# a third one with a head size that is no power of two (48), a width and vocabulary that are no multiple of 64
TINY_C = dict(model_type="gpt2", n_layer=2, n_embd=240, n_head=5, n_inner=200, vocab_size=777, n_positions=320,
              layer_norm_epsilon=3e-5, activation_function="gelu_new", scale_attn_weights=False,
              scale_attn_by_inverse_layer_idx=True)
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C}


def make_folder(tmp_path, cfg, *, seed=1, storage="float32", loud=True):
    return bt.write_random_model(tmp_path, cfg, seed=seed, storage=storage, loud=loud)


def random_prompts(cfg, lengths, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lengths]
