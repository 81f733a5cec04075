"""The generation loop's decisions, with stand-ins for the engine and the sampler (no GPU)."""
import math

import pytest

from burn_transformers_b200.cache import CacheConfig
from burn_transformers_b200.engine.generate import generate, plan_batches
from burn_transformers_b200.errors import CacheError, GenerationError
from burn_transformers_b200.sampling import (GenerationConfig, SequenceTracker, interior_unit_f32, longest_stop_suffix,
                                             sequence_stream, splitmix64, stop_decision, uniform)


class Plan:
    vocab = 50


class FakeEngine:
    """Counts what the loop asks for; its 'logits' are just the list of (slot, last token)."""
    device = "cpu"

    def __init__(self, max_tokens=64 * 8, max_slots=3, max_context=128):
        self.plan = Plan()
        self.cache_config = CacheConfig(max_tokens, max_slots, max_context)
        self.free = list(range(max_slots))
        self.live = {}
        self.steps = []
        self.released = []

    def new_sequence(self):
        slot = self.free.pop(0)
        self.live[slot] = 0
        return slot

    def release(self, slot):
        assert slot in self.live, "released twice"
        del self.live[slot]
        self.free.append(slot)
        self.released.append(slot)

    def step(self, entries):
        for e in entries:
            assert e.slot in self.live
            self.live[e.slot] += len(e.tokens)
            assert self.live[e.slot] <= self.cache_config.max_context
        self.steps.append([(e.slot, list(e.tokens), list(e.want)) for e in entries])
        return [(e.slot, e.tokens[-1]) for e in entries]


class ScriptedSampler:
    """Emits, for request r, the tokens of script[r] in order."""

    def __init__(self, script, logp=-1.0):
        self.script, self.logp, self.calls = script, logp, []

    def select(self, logits, trackers, batch_rows=None):
        self.calls.append([t.request for t in trackers])
        ids = [self.script[t.request][t.emitted] for t in trackers]
        return ids, [self.logp] * len(ids)


def test_plan_batches():
    assert plan_batches([5, 9, 17], 8, max_tokens=192, max_slots=8, max_context=128) == [[0, 1, 2]]
    assert plan_batches([5, 9, 17], 8, max_tokens=128, max_slots=8, max_context=128) == [[0, 1], [2]]
    assert plan_batches([5] * 5, 8, max_tokens=6400, max_slots=2, max_context=128) == [[0, 1], [2, 3], [4]]
    assert plan_batches([5] * 3, 8, max_tokens=6400, max_slots=8, max_context=128, max_batch=1) == [[0], [1], [2]]
    assert plan_batches([60], 5, max_tokens=64, max_slots=1, max_context=64) == [[0]]      # 60 + 5 - 1 = 64 fits
    with pytest.raises(GenerationError, match="need 65 positions"):
        plan_batches([60], 6, max_tokens=640, max_slots=1, max_context=64)
    with pytest.raises(GenerationError, match="the cache holds"):
        plan_batches([100], 8, max_tokens=64, max_slots=1, max_context=128)
    with pytest.raises(GenerationError, match="empty"):
        plan_batches([3, 0], 8, max_tokens=640, max_slots=4, max_context=128)


def test_unequal_prompts_one_prefill_then_single_tokens():
    engine = FakeEngine()
    script = {0: [1, 2, 3, 4], 1: [5, 6, 7, 8], 2: [9, 10, 11, 12]}
    out = generate(engine, [[1, 2, 3], [4], [5, 6, 7, 8, 9]], GenerationConfig(max_new_tokens=3),
                   sampler=ScriptedSampler(script))
    assert [o.token_ids for o in out] == [[1, 2, 3], [5, 6, 7], [9, 10, 11]]
    assert all(o.finish_reason.kind == "length" for o in out)
    assert [o.prompt_length for o in out] == [3, 1, 5]
    first = engine.steps[0]
    assert [len(t) for _, t, _ in first] == [3, 1, 5] and [w for _, _, w in first] == [[2], [0], [4]]
    # the last emitted token is never fed back: 1 prefill + 2 decode steps for 3 new tokens
    assert len(engine.steps) == 3 and all(len(t) == 1 for s in engine.steps[1:] for _, t, _ in s)
    assert engine.steps[1] == [(0, [1], [0]), (1, [5], [0]), (2, [9], [0])]
    assert sorted(engine.released) == [0, 1, 2] and not engine.live


def test_sequences_that_end_earlier_leave_the_batch():
    engine = FakeEngine()
    script = {0: [7, 49, 1, 1, 1], 1: [3, 3, 3, 3, 3], 2: [49, 2, 2, 2, 2]}
    sampler = ScriptedSampler(script)
    seen = []
    out = generate(engine, [[1], [2], [3]], GenerationConfig(max_new_tokens=5, eos_token_ids=[49]), sampler=sampler,
                   on_token=seen.append)
    assert out[2].token_ids == [49] and out[2].finish_reason.kind == "end_of_sequence" \
        and out[2].finish_reason.token_id == 49
    assert out[0].token_ids == [7, 49] and out[1].token_ids == [3] * 5 and out[1].finish_reason.kind == "length"
    assert sampler.calls == [[0, 1, 2], [0, 1], [1], [1], [1]]
    # a finished sequence is in no later step
    assert [[slot for slot, _, _ in s] for s in engine.steps] == [[0, 1, 2], [0, 1], [1], [1], [1]]
    assert [(t.sequence, t.step, t.token_id) for t in seen][:4] == [(0, 0, 7), (1, 0, 3), (2, 0, 49), (0, 1, 49)]
    assert seen[2].finish_reason.kind == "end_of_sequence" and seen[0].finish_reason is None


def test_batches_one_after_another_reuse_slots():
    engine = FakeEngine(max_slots=2)
    script = {r: [r + 1] * 4 for r in range(5)}
    out = generate(engine, [[1, 2]] * 5, GenerationConfig(max_new_tokens=2), sampler=ScriptedSampler(script))
    assert [o.token_ids for o in out] == [[r + 1] * 2 for r in range(5)]
    assert len(engine.released) == 5 and set(engine.released) == {0, 1} and not engine.live
    prefill_steps = [s for s in engine.steps if len(s[0][1]) == 2]
    assert [len(s) for s in prefill_steps] == [2, 2, 1]


def test_stop_sequences_and_min_new_tokens():
    cfg = GenerationConfig(max_new_tokens=10, stop_sequences=[[4, 5], [3, 4, 5], [9]], min_new_tokens=0)
    out = generate(FakeEngine(), [[1]], cfg, sampler=ScriptedSampler({0: [3, 4, 5, 6]}))
    r = out[0].finish_reason
    assert out[0].token_ids == [3, 4, 5] and (r.kind, r.index, r.length) == ("stop_sequence", 1, 3)
    cfg = GenerationConfig(max_new_tokens=6, stop_sequences=[[4, 5]], min_new_tokens=4)
    out = generate(FakeEngine(), [[1]], cfg, sampler=ScriptedSampler({0: [4, 5, 1, 4, 5, 7]}))
    assert out[0].token_ids == [4, 5, 1, 4, 5]     # the first match came before min_new_tokens
    assert longest_stop_suffix([1, 2, 3], [[3], [2, 3], [9, 2, 3]]) == (1, 2)
    assert stop_decision(True, 5, [5], [[5]], 0, 10).kind == "end_of_sequence"     # EOS wins over a stop sequence
    assert stop_decision(False, 5, [5], [], 0, 1).kind == "length"
    assert stop_decision(False, 5, [5], [], 0, 2) is None


def test_non_finite_score_stops_before_emission_and_slots_come_back():
    engine = FakeEngine()
    seen = []
    with pytest.raises(GenerationError, match="non-finite"):
        generate(engine, [[1], [2]], GenerationConfig(max_new_tokens=3),
                 sampler=ScriptedSampler({0: [1, 1, 1], 1: [2, 2, 2]}, logp=float("nan")), on_token=seen.append)
    assert not seen and not engine.live and sorted(engine.released) == [0, 1]


def test_capacity_preflight_and_bad_options():
    with pytest.raises(GenerationError, match="positions"):
        generate(FakeEngine(max_context=16), [[1] * 10], GenerationConfig(max_new_tokens=8), sampler=ScriptedSampler({}))
    for bad, text in [(dict(max_new_tokens=0), "max_new_tokens"), (dict(temperature=0.0), "temperature"),
                      (dict(top_k=0), "top_k"), (dict(top_k=51), "top_k"), (dict(top_p=0.0), "top_p"),
                      (dict(min_p=1.5), "min_p"), (dict(eos_token_ids=[50]), "special token 50"),
                      (dict(stop_sequences=[[]]), "stop sequences"), (dict(min_new_tokens=9, max_new_tokens=3), "min_new"),
                      (dict(repetition_penalty=-1.0), "repetition_penalty"), (dict(logit_bias={60: 1.0}), "logit_bias"),
                      (dict(strategy="beam"), "strategy"), (dict(temperature=1e-46), "temperature")]:
        with pytest.raises(GenerationError, match=text):
            GenerationConfig(**bad).validate(50)
    with pytest.raises(GenerationError, match="at least one prompt"):
        generate(FakeEngine(), [], GenerationConfig(), sampler=ScriptedSampler({}))


def test_tracker_edits():
    cfg = GenerationConfig(max_new_tokens=9, repetition_penalty=1.5, presence_penalty=0.5, frequency_penalty=0.25,
                           logit_bias={7: 2.0}, eos_token_ids=[0], min_new_tokens=2, no_repeat_ngram_size=2)
    t = SequenceTracker(0, [3, 4, 3], cfg)
    t.push(4, -0.1)
    edits = t.edits()
    assert edits[7] == (2.0, 1.0, 0.0, 0.0)
    assert edits[4] == (0.0, 1.5, 0.25 + 0.5, 0.0)        # generated once; also in the prompt for repetition
    assert edits[3] == (0.0, 1.5, 0.0, 1.0)               # prompt only: no additive penalty; "4 3" would repeat
    assert edits[0][3] == 1.0                             # end-of-sequence is banned before min_new_tokens
    t.push(9, -0.1)
    assert 0 not in t.edits()
    t2 = SequenceTracker(0, [3, 4, 3], GenerationConfig(presence_penalty=1.0, additive_penalty_scope="prompt_and_generated"))
    assert t2.edits()[3] == (0.0, 1.0, 1.0, 0.0)


def test_random_streams():
    assert splitmix64(0, 0) == 0xE220A8397B1DCDAF
    assert interior_unit_f32(0) == 2.0 ** -24 and interior_unit_f32((1 << 64) - 1) == 1 - 2.0 ** -24
    assert uniform(5, 3) == interior_unit_f32(splitmix64(5, 3))
    assert sequence_stream(5, 0) != sequence_stream(5, 1)


def test_chunked_prefill_cuts_prompts_by_columns_and_asks_logits_only_where_a_prompt_ends():
    """With a chunk size every step brings at most that many tokens of each prompt that still has some; a prompt
    that has ended sits out the later portions; logits are wanted only at each prompt's last token
    (src/generation/causal.rs:341-396 of the reference)."""
    engine = FakeEngine()
    script = {0: [1, 2], 1: [5, 6], 2: [9, 10]}
    out = generate(engine, [[1, 2, 3], [4], [5, 6, 7, 8, 9]], GenerationConfig(max_new_tokens=2),
                   sampler=ScriptedSampler(script), prefill_chunk_size=2)
    assert [o.token_ids for o in out] == [[1, 2], [5, 6], [9, 10]]
    assert engine.steps[0] == [(0, [1, 2], []), (1, [4], [0]), (2, [5, 6], [])]
    assert engine.steps[1] == [(0, [3], [0]), (2, [7, 8], [])]
    assert engine.steps[2] == [(2, [9], [0])]
    assert engine.steps[3] == [(0, [1], [0]), (1, [5], [0]), (2, [9], [0])]      # then one token each
    assert len(engine.steps) == 4 and not engine.live
    # a chunk as long as the longest prompt is the one-shot prefill
    engine = FakeEngine()
    generate(engine, [[1, 2, 3], [4]], GenerationConfig(max_new_tokens=1), sampler=ScriptedSampler({0: [1], 1: [2]}),
             prefill_chunk_size=3)
    assert engine.steps == [[(0, [1, 2, 3], [2]), (1, [4], [0])]]
    with pytest.raises(GenerationError, match="prefill_chunk_size"):
        generate(FakeEngine(), [[1]], GenerationConfig(max_new_tokens=1), sampler=ScriptedSampler({0: [1]}),
                 prefill_chunk_size=0)
