"""Schedules that serving takes and the replay tests of test_model_gpu.py do not reach, all against the plain
implementation with loud weights (a lost key or a wrong slot moves the logits):

* decode steps of more than 16 sequences (17 to 64 rows take the kernels made for them under a CUDA graph with
  programmatic dependent launch, more than 64 rows the tcgen05 product);
* one prefill shape fed several times to one engine (from the third time on it is a replayed CUDA graph), with
  other lengths behind the same shape, and more distinct shapes than the engine keeps recordings of;
* a prompt fed in portions (several tokens for a sequence that already holds some), portions that ask for no
  logits and are never waited for, a portion that ends on a page boundary, and steps that mix a fresh sequence,
  a continued one and a one-token one;
* chunked prefill in the generation loop.
"""
import numpy as np
import pytest

import engine_replay as replay
import plain_gpt2 as plain
import burn_transformers_b200 as bt
from burn_transformers_b200 import Engine, StepEntry
from tiny_configs import CONFIGS, make_folder, random_prompts

pytestmark = pytest.mark.gpu

TOL = {"float32": 1e-4, "bfloat16": 3e-2}      # as in test_model_gpu.py
# a third configuration with the head size of the published models (64), so that the tensor-core kernels run
HEAD64 = dict(model_type="gpt2", n_layer=2, n_embd=128, n_head=2, n_inner=384, vocab_size=331, n_positions=192,
              layer_norm_epsilon=1e-5, activation_function="gelu_new")
ALL = dict(CONFIGS, H=HEAD64)


def references(folder, seqs):
    pcfg, pw = plain.load_model(folder)
    rounded = {k: (plain.round_to_bf16(v) if v.ndim == 2 else v) for k, v in pw.items()}
    return {"float32": [plain.logits(pcfg, pw, s) for s in seqs],
            "bfloat16": [plain.logits(pcfg, rounded, s, quant=plain.round_to_bf16) for s in seqs]}


@pytest.fixture(scope="module", params=["A", "B", "H"])
def model(request, tmp_path_factory):
    name = request.param
    folder = make_folder(tmp_path_factory.mktemp(f"sched{name}"), ALL[name], seed=23, storage="float32", loud=True)
    return name, ALL[name], folder


# ---- many sequences -----------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("batch", [17, 33, 64, 70])
def test_decoding_many_sequences_together(model, dtype, batch):
    name, cfg, folder = model
    if name == "B" and batch in (33, 70):
        pytest.skip("one large and one small batch are enough for this configuration")
    lengths = [14 + (i % 3) + (9 if i % 7 == 0 else 0) for i in range(batch)]
    prompts = [4 + (i % 5) for i in range(batch)]
    seqs = random_prompts(cfg, lengths, seed=batch)
    ref = references(folder, seqs)[dtype]
    engine = Engine.from_folder(folder, dtype, max_tokens=64 * batch, max_slots=batch)
    got = replay.batches(engine, seqs, [list(range(batch))], prompts)
    assert len(got) == sum(lengths)
    err, where = replay.worst_error(got, ref)
    assert err < TOL[dtype], f"{batch} sequences, {dtype}: {err:.3e} at {where}"
    if engine.use_graphs:
        sizes = sorted(n for (n, _), g in engine._graphs.items())
        assert sizes[-1] == batch and len(sizes) >= 2        # the batch shrank as the shorter requests ended


# ---- a prefill shape that repeats ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_repeated_prefill_shape_is_right_every_time(model, dtype):
    """The same shape (tokens, sequences, longest run, wanted rows) five times: the first two run kernel by kernel,
    the later ones replay a recording.  The lengths behind the shape change (the same total cut differently), and
    so do the slots and pages."""
    name, cfg, folder = model
    engine = Engine.from_folder(folder, dtype, max_tokens=64 * 8)
    cuts = [(20, 9, 5), (20, 5, 9), (20, 13, 1), (20, 7, 7), (20, 1, 13)]        # all: 34 tokens, 3 sequences, longest 20
    held = []
    for round_index, cut in enumerate(cuts):
        seqs = random_prompts(cfg, list(cut), seed=100 + round_index)
        ref = references(folder, seqs)[dtype]
        slots = [engine.new_sequence() for _ in seqs]
        logits = engine.step([StepEntry(s, seq, list(range(len(seq)))) for s, seq in zip(slots, seqs)])
        host = logits.cpu().double().numpy()
        at = 0
        for r, seq in enumerate(seqs):
            err = np.abs(host[at:at + len(seq)] - ref[r]).max() / np.abs(ref[r]).max()
            assert err < TOL[dtype], f"round {round_index}, request {r}: {err:.3e}"
            at += len(seq)
        # keep one sequence of every round alive, so that later rounds get other slots and pages
        held.append(slots[0])
        for s in slots[1:]:
            engine.release(s)
    if engine.use_graphs:
        assert len(engine._shape_graphs) == 1 and next(iter(engine._shape_graphs.values())).graph is not None
    for s in held:
        engine.release(s)
    engine.cache.check()


def test_more_shapes_than_recordings_are_kept(model):
    """Ten distinct shapes, each met three times: the engine keeps the eight most recent recordings and every
    result is right, also for a shape whose recording was dropped and made again."""
    name, cfg, folder = model
    engine = Engine.from_folder(folder, "bfloat16", max_tokens=64 * 4)
    shapes = [(3 + i, 2 + (i % 2)) for i in range(10)]
    seqs_by_shape = {shape: random_prompts(cfg, list(shape), seed=sum(shape)) for shape in shapes}
    ref = {shape: references(folder, seqs)["bfloat16"] for shape, seqs in seqs_by_shape.items()}
    for round_index in range(3):
        for shape in shapes:
            seqs = seqs_by_shape[shape]
            got = replay.batches(engine, seqs, [[0, 1]], [len(s) for s in seqs])
            err, where = replay.worst_error(got, ref[shape])
            assert err < TOL["bfloat16"], f"round {round_index}, shape {shape}: {err:.3e} at {where}"
    if engine.use_graphs:
        assert len(engine._shape_graphs) == engine.max_shape_graphs


# ---- prompts in portions ------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_prompt_fed_in_portions(model, dtype):
    """40 + 24 + 2 + 21 tokens (the second portion ends on the page boundary at 64, the third brings two tokens),
    then one by one: several tokens for a sequence that already holds some take the paged prefill kernels."""
    name, cfg, folder = model
    seqs = random_prompts(cfg, [100], seed=3)
    ref = references(folder, seqs)[dtype]
    engine = Engine.from_folder(folder, dtype, max_tokens=64 * 4)
    seq = seqs[0]
    slot = engine.new_sequence()
    got, at = {}, 0
    for n in (40, 24, 2, 21):
        logits = engine.step([StepEntry(slot, seq[at:at + n], list(range(n)))])
        for i, row in enumerate(logits.cpu().double().numpy()):
            got[(0, at + i)] = row
        at += n
    for p in range(at, len(seq)):
        got[(0, p)] = engine.step([StepEntry(slot, [seq[p]], [0])]).cpu().double().numpy()[0]
    engine.release(slot)
    err, where = replay.worst_error(got, ref)
    assert len(got) == len(seq) and err < TOL[dtype], f"portions {dtype}: {err:.3e} at {where}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_that_nobody_waits_for(model, dtype):
    """Portions that ask for no logits return nothing the host could wait for: four such steps are queued back to
    back (the same shape twice, so that a recording is replayed), and only the last portion's logits are read.
    The integers of a step (tokens, positions, page tables) must reach the device as that step's, whatever the
    host has written for later steps meanwhile."""
    name, cfg, folder = model
    seqs = random_prompts(cfg, [97, 75], seed=8)
    ref = references(folder, seqs)[dtype]
    engine = Engine.from_folder(folder, dtype, max_tokens=64 * 4)
    slots = [engine.new_sequence() for _ in seqs]
    fed = [0, 0]
    for portion in ((30, 20), (2, 2), (30, 20), (2, 2), (30, 20)):
        entries = [StepEntry(slots[r], seqs[r][fed[r]:fed[r] + n], []) for r, n in enumerate(portion)]
        assert engine.step(entries) is None
        for r, n in enumerate(portion):
            fed[r] += n
    entries = [StepEntry(slots[r], seqs[r][fed[r]:], list(range(len(seqs[r]) - fed[r]))) for r in range(2)]
    host = engine.step(entries).cpu().double().numpy()
    at = 0
    for r in range(2):
        n = len(seqs[r]) - fed[r]
        err = np.abs(host[at:at + n] - ref[r][fed[r]:]).max() / np.abs(ref[r]).max()
        assert err < TOL[dtype], f"request {r}: {err:.3e}"
        at += n
    for s in slots:
        engine.release(s)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_step_that_mixes_fresh_continued_and_one_token_sequences(model, dtype):
    name, cfg, folder = model
    seqs = random_prompts(cfg, [70, 33, 50], seed=12)
    ref = references(folder, seqs)[dtype]
    engine = Engine.from_folder(folder, dtype, max_tokens=64 * 6)
    got = {}

    def run(pieces):
        """pieces: (request, slot, first, count); logits wanted everywhere."""
        logits = engine.step([StepEntry(slot, seqs[r][a:a + n], list(range(n))) for r, slot, a, n in pieces])
        host, at = logits.cpu().double().numpy(), 0
        for r, _, a, n in pieces:
            for i in range(n):
                got[(r, a + i)] = host[at + i]
            at += n

    s0, s1 = engine.new_sequence(), engine.new_sequence()
    run([(0, s0, 0, 45), (1, s1, 0, 10)])
    s2 = engine.new_sequence()
    run([(0, s0, 45, 1), (1, s1, 10, 23), (2, s2, 0, 50)])        # one token, a continued run, a fresh prompt
    run([(0, s0, 46, 24)])
    for s in (s0, s1, s2):
        engine.release(s)
    err, where = replay.worst_error(got, ref)
    assert len(got) == sum(len(s) for s in seqs) and err < TOL[dtype], f"mixed {dtype}: {err:.3e} at {where}"
    engine.cache.check()


# ---- chunked prefill in the generation loop -----------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_chunked_prefill_generates_what_one_shot_prefill_generates(model, dtype):
    """(src/generation/causal_tests.rs:526 of the reference: chunked == one-shot.)  In 32-bit the tokens are also
    those of the plain implementation."""
    name, cfg, folder = model
    prompts = random_prompts(cfg, [37, 5, 64, 18], seed=31)
    config = bt.GenerationConfig(max_new_tokens=6)
    engine = Engine.from_folder(folder, dtype, max_tokens=64 * 8)
    one_shot = bt.generate(engine, prompts, config)
    chunked = bt.generate(engine, prompts, config, prefill_chunk_size=16)
    tiny = bt.generate(engine, prompts, config, prefill_chunk_size=1)
    if dtype == "float32":
        pcfg, pw = plain.load_model(folder)
        want = [plain.generate(pcfg, pw, p, 6)[0] for p in prompts]
        assert [o.token_ids for o in one_shot] == want
        assert [o.token_ids for o in chunked] == want and [o.token_ids for o in tiny] == want
    for a, b, c in zip(one_shot, chunked, tiny):
        # (bfloat16: the same kernels see the same rows up to the order of summation; compare what they are sure of)
        assert np.allclose(a.log_probabilities[:1], b.log_probabilities[:1], atol=5e-2)
        assert np.allclose(a.log_probabilities[:1], c.log_probabilities[:1], atol=5e-2)
    engine.cache.check()
    assert engine.cache.slots.held == 0
