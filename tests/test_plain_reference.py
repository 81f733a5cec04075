"""The plain implementation against the reference project's committed fixture, and its own parts."""
import json
import math
from pathlib import Path

import numpy as np
import pytest

import plain_gpt2 as plain

GOLDEN = json.loads((Path(__file__).parent / "golden" / "gpt2_tiny_reference.json").read_text())
MASK = (1 << 64) - 1


def fixture_weights():
    """The fixture's generated weights (src/models/gpt2/prepare_reference.py:21-41 of the
    reference): tensors in sorted name order, a 64-bit xorshift per tensor."""
    weights = {}
    for index, name in enumerate(sorted(GOLDEN["parameter_shapes"])):
        shape = GOLDEN["parameter_shapes"][name]
        state = (GOLDEN["seed"] ^ ((index + 1) * 0x9E3779B97F4A7C15)) & MASK
        is_scale = name.endswith(".weight") and (".ln_" in name or name.startswith("ln_f."))
        shift = 32 if name.endswith(".bias") else 23 if name.endswith("mlp.c_fc.weight") else 29
        values = []
        for _ in range(int(np.prod(shape))):
            state ^= (state << 13) & MASK
            state ^= state >> 7
            state ^= (state << 17) & MASK
            value = ((state >> 40) - (1 << 23)) / (1 << shift)
            values.append(1.0 + value if is_scale else value)
        weights[name] = np.array(values, dtype=np.float32).astype(np.float64).reshape(shape)
    return weights


@pytest.mark.parametrize("act", ["gelu_new", "gelu"])
def test_plain_matches_reference_fixture(act):
    cfg = dict(GOLDEN["config"], activation_function=act, causal=True)
    w = fixture_weights()
    ref = GOLDEN["references"][act]
    for row, (ids, mask) in enumerate(zip(GOLDEN["input_ids"], GOLDEN["token_mask"])):
        taps = {}
        got = plain.logits(cfg, w, ids, key_valid=mask, taps=taps)
        # tolerances of src/models/gpt2/model_tests.rs:185-204: 2e-6 logits and MLP, 3e-6 hidden
        assert np.abs(got - np.array(ref["logits"][row])).max() < 2e-6
        assert np.abs(taps["final_norm"] - np.array(ref["final_norm"][row])).max() < 3e-6
        assert np.abs(taps["embedding"] - np.array(ref["embedding"][row])).max() < 3e-6
        for layer in range(cfg["n_layer"]):
            want = np.array(ref["mlp_outputs"][f"mlp_{layer}"][row])
            assert np.abs(taps["mlp"][layer] - want).max() < 2e-6


def test_padded_key_is_the_same_as_a_shorter_sequence():
    cfg = dict(GOLDEN["config"], activation_function="gelu_new", causal=True)
    w = fixture_weights()
    ids = GOLDEN["input_ids"][1]
    padded = plain.logits(cfg, w, ids, key_valid=[1, 1, 1, 0])
    short = plain.logits(cfg, w, ids[:3])
    assert np.abs(padded[:3] - short).max() < 1e-12


def test_scale_flags_equal_scaled_queries():
    """Both score-scale flags, checked as the reference does: dividing the scores by c is
    the same as dividing the queries by c (src/models/gpt2/model_tests.rs:1338-1387)."""
    cfg = dict(GOLDEN["config"], activation_function="gelu_new", causal=True)
    w = fixture_weights()
    ids = GOLDEN["input_ids"][0]
    d, hd = cfg["n_embd"], cfg["n_embd"] // cfg["n_head"]
    base = dict(cfg, scale_attn_weights=False, scale_attn_by_inverse_layer_idx=False)
    for flags in [dict(scale_attn_weights=True, scale_attn_by_inverse_layer_idx=True),
                  dict(scale_attn_weights=False, scale_attn_by_inverse_layer_idx=True)]:
        want = plain.logits(dict(cfg, **flags), w, ids)
        w2 = {k: v.copy() for k, v in w.items()}
        for layer in range(cfg["n_layer"]):
            c = (math.sqrt(hd) if flags["scale_attn_weights"] else 1.0) * (layer + 1)
            w2[f"h.{layer}.attn.c_attn.weight"][:, :d] /= c
            w2[f"h.{layer}.attn.c_attn.bias"][:d] /= c
        got = plain.logits(base, w2, ids)
        assert np.abs(got - want).max() < 1e-12


def test_all_excluded_row_is_zero():
    p = plain.softmax_rows(np.zeros((2, 3)), np.array([[True, True, True], [False, True, True]]))
    assert p[0].sum() == 0 and p[1, 0] == 1.0


def test_bottom_right_causal_alignment():
    ex = plain.excluded(2, 5)
    assert ex.tolist() == [[False, False, False, False, True], [False] * 5]
    exw = plain.excluded(1, 5, window=2)
    assert exw.tolist() == [[True, True, True, False, False]]


def test_splitmix_and_unit():
    # first outputs of the classic SplitMix64 sequence started at 0
    assert plain.splitmix64(0, 0) == 0xE220A8397B1DCDAF
    assert plain.splitmix64(0, 1) == 0x6E789E6AA1B965F4
    u = plain.interior_unit(plain.splitmix64(7, 3))
    assert 0.0 < u < 1.0
    assert plain.interior_unit(0) == 2.0 ** -24
    assert plain.interior_unit(MASK) == 1.0 - 2.0 ** -24


def test_filters():
    z = np.array([1.0, 3.0, 3.0, 0.5, 2.0])
    assert np.isfinite(plain.top_k_filter(z, 1)).tolist() == [False, True, True, False, False]
    assert np.isfinite(plain.top_k_filter(z, 3)).tolist() == [False, True, True, False, True]
    kept = np.isfinite(plain.top_p_filter(np.log(np.array([0.5, 0.3, 0.15, 0.05])), 0.79))
    assert kept.tolist() == [True, True, False, False]
    kept = np.isfinite(plain.top_p_filter(np.log(np.array([0.5, 0.3, 0.15, 0.05])), 0.81))
    assert kept.tolist() == [True, True, True, False]
    kept = np.isfinite(plain.min_p_filter(np.log(np.array([0.5, 0.3, 0.15, 0.04])), 0.1))
    assert kept.tolist() == [True, True, True, False]


def test_select_inverse_cdf():
    z = np.log(np.array([0.1, 0.2, 0.3, 0.4]))
    assert plain.select(z, sample=True, u=0.05)[0] == 0
    assert plain.select(z, sample=True, u=0.25)[0] == 1
    assert plain.select(z, sample=True, u=0.999)[0] == 3
    tok, lp = plain.select(z, sample=False)
    assert tok == 3 and abs(lp - math.log(0.4)) < 1e-12


def test_bf16_rounding():
    x = np.array([1.0, 1.0 + 2 ** -9, 1.0 + 2 ** -8, 3.1415926, -0.3])
    r = plain.round_to_bf16(x)
    assert r[0] == 1.0 and r[1] == 1.0 and r[2] == 1.0  # ties go to the even mantissa
    assert abs(r[3] - 3.140625) < 1e-12
