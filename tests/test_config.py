"""Configuration and registry (no GPU)."""
import json

import pytest

import burn_transformers_b200 as bt
from burn_transformers_b200.config import Gpt2Config, architecture_for, config_from_folder
from burn_transformers_b200.errors import ConfigError, UnsupportedArchitecture


def test_defaults_are_gpt2_small():
    c = Gpt2Config.from_dict({"model_type": "gpt2"})
    assert (c.vocab_size, c.n_embd, c.n_layer, c.n_head, c.n_positions) == (50257, 768, 12, 12, 1024)
    assert c.intermediate_size == 3072 and c.head_dim == 64 and c.activation_function == "gelu_new"
    assert c.layer_norm_epsilon == 1e-5 and c.scale_attn_weights and not c.scale_attn_by_inverse_layer_idx


def test_aliases_and_unknown_keys():
    c = Gpt2Config.from_dict({"hidden_size": 96, "num_hidden_layers": 3, "num_attention_heads": 3,
                              "max_position_embeddings": 77, "resid_pdrop": 0.1, "summary_type": "cls_index"})
    assert (c.n_embd, c.n_layer, c.n_head, c.n_positions) == (96, 3, 3, 77)


def test_n_inner_and_scale():
    c = Gpt2Config.from_dict({"n_embd": 96, "n_head": 3, "n_inner": 320, "scale_attn_by_inverse_layer_idx": True})
    assert c.intermediate_size == 320
    assert c.score_scale(0) == pytest.approx(32 ** -0.5)
    assert c.score_scale(2) == pytest.approx(32 ** -0.5 / 3)
    c2 = Gpt2Config.from_dict({"scale_attn_weights": False})
    assert c2.score_scale(5) == 1.0


@pytest.mark.parametrize("patch, field", [
    ({"model_type": "llama"}, "model_type"),
    ({"vocab_size": 0}, "vocab_size"),
    ({"n_embd": 2 ** 31}, "n_embd"),
    ({"n_layer": 0}, "n_layer"),
    ({"n_layer": (1 << 18) + 1}, "n_layer"),
    ({"n_embd": 100, "n_head": 3}, "n_head"),
    ({"layer_norm_epsilon": 0.0}, "layer_norm_epsilon"),
    ({"initializer_range": float("inf")}, "initializer_range"),
    ({"reorder_and_upcast_attn": True}, "reorder_and_upcast_attn"),
    ({"add_cross_attention": True}, "add_cross_attention"),
    ({"tie_word_embeddings": False}, "tie_word_embeddings"),
    ({"activation_function": "relu"}, "activation_function"),
    ({"n_inner": 0}, "n_inner"),
    ({"n_head": "12"}, "n_head"),
    ({"scale_attn_weights": 1}, "scale_attn_weights"),
])
def test_errors_name_the_field(patch, field):
    with pytest.raises(ConfigError) as info:
        Gpt2Config.from_dict(patch)
    assert info.value.field == field
    assert str(info.value).startswith(f"gpt2.{field}: ")


def test_first_invalid_extent_is_named():
    with pytest.raises(ConfigError) as info:
        Gpt2Config.from_dict({"n_head": 0, "vocab_size": 0})
    assert info.value.field == "vocab_size"


def test_registry(tmp_path):
    assert "gpt2" in bt.supported_model_types()
    assert architecture_for("gpt2").config_class is Gpt2Config
    with pytest.raises(UnsupportedArchitecture) as info:
        architecture_for("mamba2")
    assert "supported values" in str(info.value) and "gpt2" in str(info.value)
    (tmp_path / "config.json").write_text(json.dumps({"text_config": {"model_type": "gpt2", "n_layer": 2}}))
    arch, config = config_from_folder(tmp_path)
    assert arch.name == "gpt2" and config.n_layer == 2
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        config_from_folder(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps({"n_layer": 2}))
    with pytest.raises(ConfigError) as info:
        config_from_folder(tmp_path)
    assert info.value.field == "model_type"


def test_plan_has_every_tensor_once():
    plan = architecture_for("gpt2").build(Gpt2Config.from_dict({"n_layer": 2, "n_embd": 64, "n_head": 4,
                                                                 "vocab_size": 512, "n_positions": 128}))
    names = plan.weights.tensors
    assert len(names) == 4 + 12 * 2
    assert names["h.1.attn.c_attn.weight"].shape == (64, 192)
    assert names["h.0.mlp.c_fc.weight"].shape == (64, 256)
    assert names["wpe.weight"].shape == (128, 64)
    assert [c.block for c in plan.schedule] == [0, 1]


@pytest.mark.parametrize("patch, field", [
    ({"n_embd": 1028, "n_head": 2}, "n_head"),      # head size 514: more than the attention kernels take
    ({"causal": False}, "causal"),                   # a cached engine decodes causally
])
def test_what_the_engine_does_not_run_is_refused_by_field_when_the_model_is_built(patch, field):
    """config.json may ask for things that parse and validate but that this engine cannot execute; the builder
    refuses them as a configuration error that names the field, never as a bare exception from a part."""
    from burn_transformers_b200.models.gpt2 import build_gpt2
    config = Gpt2Config.from_dict(dict({"model_type": "gpt2", "n_layer": 1, "vocab_size": 32, "n_positions": 16}, **patch))
    with pytest.raises(ConfigError) as info:
        build_gpt2(config)
    assert info.value.field == field and str(info.value).startswith(f"gpt2.{field}: ")


@pytest.mark.parametrize("n_embd, n_head", [(12, 3), (15, 3), (7, 1), (36, 3), (40, 5)])
def test_every_head_size_the_configuration_allows_builds(n_embd, n_head):
    """The reference asks only that n_head divide n_embd (src/models/gpt2.rs:258-318); its own fixture has head size 4."""
    from burn_transformers_b200.models.gpt2 import build_gpt2
    plan = build_gpt2(Gpt2Config.from_dict({"model_type": "gpt2", "n_layer": 1, "vocab_size": 19, "n_positions": 16,
                                            "n_embd": n_embd, "n_head": n_head}))
    assert plan.blocks[0].mixer.head_dim == n_embd // n_head
