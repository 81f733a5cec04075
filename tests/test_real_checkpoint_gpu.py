"""Opt-in check against a real GPT-2 checkpoint on this machine, in the manner of the reference's own
(src/models/gpt2/model_tests.rs:981-1095 and src/models/gpt2/README.md:38-92 of NoahIsCool/burn-transformers).

Nothing is downloaded.  With `GPT2_CHECKPOINT` naming a folder that holds `config.json` and `model.safetensors`:

* the engine's 32-bit logits at the last token of two prompts are compared with the plain implementation over the whole
  vocabulary, within the reference's bounds: `1e-4 + 1e-5 * abs(reference)` for logits and
  `1e-5 + 1e-4 * abs(reference)` for probabilities;
* with `GPT2_REFERENCE` also naming the JSON file that the reference's `prepare_reference.py` writes
  (`input_ids`, `reference.logits` from an independent PyTorch model), the engine is compared with those numbers as well.

Without the variables the tests are skipped.
"""
import json
import os

import numpy as np
import pytest

import plain_gpt2 as plain
from burn_transformers_b200 import Engine, StepEntry

pytestmark = pytest.mark.gpu

CHECKPOINT = os.environ.get("GPT2_CHECKPOINT")
REFERENCE = os.environ.get("GPT2_REFERENCE")
needs_checkpoint = pytest.mark.skipif(not CHECKPOINT, reason="set GPT2_CHECKPOINT to a local GPT-2 folder to run this check")

# two short prompts as token ids (any ids below the vocabulary will do: the check is numerical)
PROMPTS = [[464, 1175, 15436, 422, 262, 614, 1596, 2624, 284, 262, 614, 1596], [464, 3427, 4631, 373, 3170, 287, 262, 614, 1248]]


def _probabilities(row):
    z = np.asarray(row, dtype=np.float64)
    z = np.exp(z - z.max())
    return z / z.sum()


def _engine_last_logits(engine, prompts):
    out = []
    for ids in prompts:
        slot = engine.new_sequence()
        try:
            out.append(engine.step([StepEntry(slot, list(ids), [len(ids) - 1])]).float().cpu().numpy()[0])
        finally:
            engine.release(slot)
    return out


def _assert_close(got, want, what):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    worst = np.abs(got - want).max()
    assert (np.abs(got - want) <= 1e-4 + 1e-5 * np.abs(want)).all(), f"{what}: largest logit error {worst:.3e}"
    p_got, p_want = _probabilities(got), _probabilities(want)
    p_worst = np.abs(p_got - p_want).max()
    assert (np.abs(p_got - p_want) <= 1e-5 + 1e-4 * p_want).all(), f"{what}: largest probability error {p_worst:.3e}"


@needs_checkpoint
def test_last_token_logits_of_a_real_checkpoint_match_the_plain_implementation():
    cfg, weights = plain.load_model(CHECKPOINT)
    engine = Engine.from_folder(CHECKPOINT, "float32", max_tokens=64 * 2)
    got = _engine_last_logits(engine, PROMPTS)
    for ids, row in zip(PROMPTS, got):
        want = plain.logits(cfg, weights, ids)[-1]
        _assert_close(row, want, f"prompt of {len(ids)} tokens")


@needs_checkpoint
@pytest.mark.skipif(not REFERENCE, reason="set GPT2_REFERENCE to the JSON file of the reference's prepare_reference.py")
def test_last_token_logits_of_a_real_checkpoint_match_the_recorded_pytorch_numbers():
    with open(REFERENCE) as handle:
        fixture = json.load(handle)
    prompts = fixture["input_ids"]
    recorded = fixture["reference"]["logits"]          # [batch][position][vocab] or [batch][vocab] for the last position
    engine = Engine.from_folder(CHECKPOINT, "float32", max_tokens=64 * max(1, -(-max(map(len, prompts)) // 64)))
    got = _engine_last_logits(engine, prompts)
    for i, row in enumerate(got):
        want = np.asarray(recorded[i])
        _assert_close(row, want[-1] if want.ndim == 2 else want, f"recorded prompt {i}")
