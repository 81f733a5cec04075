"""Extracts the golden vectors of the reference project's committed GPT-2 fixture.

The reference (NoahIsCool/burn-transformers) commits
`src/models/gpt2/fixtures/tiny_reference.json`: outputs of an independent
PyTorch GPT-2 on a tiny configuration whose weights come from a deterministic
generator (`src/models/gpt2/prepare_reference.py:21-41`, mirrored in
`src/models/gpt2/model_tests.rs:50-86`).  Its Rust model code cannot be compiled
here, so these vectors are what anchors `tests/plain_gpt2.py`.

    python tests/golden/make_gpt2_tiny_reference.py REFERENCE_ROOT

writes `tests/golden/gpt2_tiny_reference.json` with the configuration, the
inputs, and for both activations the logits, the final-norm states and the
per-block MLP outputs, as the fixture holds them (numbers unchanged).
"""
import json
import sys
from pathlib import Path


def main():
    root = Path(sys.argv[1])
    src = json.loads((root / "src/models/gpt2/fixtures/tiny_reference.json").read_text())
    keep = ("vocab_size", "n_positions", "n_embd", "n_layer", "n_head", "n_inner",
            "layer_norm_epsilon", "scale_attn_weights", "scale_attn_by_inverse_layer_idx",
            "model_type", "tie_word_embeddings", "initializer_range")
    out = {
        "source": "src/models/gpt2/fixtures/tiny_reference.json of NoahIsCool/burn-transformers",
        "versions": src["versions"],
        "seed": src["seed"],
        "config": {k: src["config"][k] for k in keep},
        "parameter_shapes": src["parameter_shapes"],
        "input_ids": src["input_ids"],
        "token_mask": src["token_mask"],
        "references": {
            name: {
                "logits": ref["logits"],
                "final_norm": ref["hidden_states"][-1],
                "embedding": ref["hidden_states"][0],
                "mlp_outputs": ref["mlp_outputs"],
            }
            for name, ref in src["references"].items()
        },
    }
    target = Path(__file__).parent / "gpt2_tiny_reference.json"
    target.write_text(json.dumps(out, sort_keys=True, separators=(",", ":")) + "\n")
    print(target)


if __name__ == "__main__":
    main()
