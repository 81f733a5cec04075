"""The engine itself against the reference project's own numbers.

The reference anchors its GPT-2 on an independent PyTorch model and commits that model's outputs for a tiny
configuration (src/models/gpt2/fixtures/tiny_reference.json: vocabulary 19, width 12, three heads of size 4,
feed-forward width 17; used at src/models/gpt2/model_tests.rs:152-206).  Here the fixture's weights are
regenerated, written as a model folder and run through `Engine.step` in true 32-bit: as a ragged batch (the
fixture's second row has one padded column, so the engine is given its three real tokens), each row alone, and
token by token.  The bound is the reference's 32-bit cross-backend bound, 2e-5 + 2e-5 * scale
(tests/backend_parity.rs:251).

A second, opt-in test takes a real GPT-2 folder when the environment offers one, as
src/models/gpt2/model_tests.rs:981-1095 does.
"""
import json
import os

import numpy as np
import pytest
import torch

import engine_replay as replay
import plain_gpt2 as plain
from burn_transformers_b200 import Engine, StepEntry
from burn_transformers_b200.weights import safetensors_io
from test_plain_reference import GOLDEN, fixture_weights

pytestmark = pytest.mark.gpu


def fixture_folder(tmp_path, activation):
    config = dict(GOLDEN["config"], activation_function=activation)
    (tmp_path / "config.json").write_text(json.dumps(config))
    tensors = {name: torch.from_numpy(value.astype(np.float32)) for name, value in fixture_weights().items()}
    safetensors_io.write_file(tmp_path / "model.safetensors", tensors)
    return tmp_path


def fixture_requests():
    """The fixture's rows without their padding: the key mask of a right-padded row is a shorter sequence."""
    return [[t for t, keep in zip(ids, mask) if keep] for ids, mask in zip(GOLDEN["input_ids"], GOLDEN["token_mask"])]


def within_reference_bound(got, want):
    want = np.asarray(want, dtype=np.float64)
    scale = np.abs(want).max()
    return np.abs(np.asarray(got, dtype=np.float64) - want).max() <= 2e-5 + 2e-5 * scale


@pytest.mark.parametrize("activation", ["gelu_new", "gelu"])
def test_engine_reproduces_the_reference_fixture_in_32_bit(tmp_path, activation):
    folder = fixture_folder(tmp_path, activation)
    engine = Engine.from_folder(folder, "float32", max_tokens=256)
    seqs = fixture_requests()
    want = GOLDEN["references"][activation]["logits"]
    # the ragged batch in one step
    slots = [engine.new_sequence() for _ in seqs]
    logits = engine.step([StepEntry(s, seq, list(range(len(seq)))) for s, seq in zip(slots, seqs)]).cpu().numpy()
    at = 0
    for row, seq in enumerate(seqs):
        assert within_reference_bound(logits[at:at + len(seq)], want[row][:len(seq)]), f"batch, row {row}"
        at += len(seq)
    for s in slots:
        engine.release(s)
    # each row alone, and with all but its first token fed one by one
    for schedule in (replay.whole, lambda e, s: replay.tail_one_by_one(e, s, tail=10 ** 6)):
        got = schedule(engine, seqs)
        for (row, position), values in got.items():
            assert within_reference_bound(values, want[row][position]), f"row {row}, position {position}"
    engine.cache.check()


def test_engine_runs_the_fixture_configuration_in_bfloat16(tmp_path):
    """Head size 4 is no multiple of any tile: bfloat16 takes the kernels that read element by element."""
    folder = fixture_folder(tmp_path, "gelu_new")
    engine = Engine.from_folder(folder, "bfloat16", max_tokens=256)
    seqs = fixture_requests()
    got = replay.tail_one_by_one(engine, seqs, tail=2)
    want = GOLDEN["references"]["gelu_new"]["logits"]
    scale = max(np.abs(np.asarray(w)).max() for w in want)
    worst = max(np.abs(values - np.asarray(want[row][position])).max() for (row, position), values in got.items())
    assert worst < 3e-2 * scale


@pytest.mark.skipif(not os.environ.get("GPT2_CHECKPOINT"), reason="set GPT2_CHECKPOINT to a GPT-2 folder "
                    "(config.json, model.safetensors) to compare the engine with the plain implementation on real weights")
def test_real_checkpoint_last_token_logits():
    """Last-token logits over the whole vocabulary, 32-bit engine against the plain implementation, within
    1e-4 + 1e-5 * |reference| (src/models/gpt2/model_tests.rs:981-1095, src/models/gpt2/README.md:38-92).
    GPT2_PROMPT_IDS may give the token ids as comma-separated integers; without it 24 ids spread over the vocabulary
    are used."""
    folder = os.environ["GPT2_CHECKPOINT"]
    cfg, weights = plain.load_model(folder)
    if os.environ.get("GPT2_PROMPT_IDS"):
        ids = [int(t) for t in os.environ["GPT2_PROMPT_IDS"].split(",")]
    else:
        ids = [(i * 7919 + 13) % cfg["vocab_size"] for i in range(24)]
    want = plain.logits(cfg, weights, ids)[-1]
    engine = Engine.from_folder(folder, "float32", max_tokens=64 * (1 + len(ids) // 64))
    slot = engine.new_sequence()
    got = engine.step([StepEntry(slot, ids, [len(ids) - 1])]).cpu().double().numpy()[0]
    assert np.all(np.abs(got - want) <= 1e-4 + 1e-5 * np.abs(want))
    assert int(np.argmax(got)) == int(np.argmax(want))
