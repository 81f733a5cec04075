"""Generation through the entry points, and trace replay as a program."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import plain_gpt2 as plain
import burn_transformers_b200 as bt
from burn_transformers_b200 import (AutoCausalLm, AutoLoadOptions, CausalGenerationRequest, GenerationConfig,
                                    generate_causal, generate_causal_streaming)
from burn_transformers_b200.sampling import sequence_stream
from tiny_configs import TINY_A, TINY_B, make_folder, random_prompts

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def model_a(tmp_path_factory):
    folder = make_folder(tmp_path_factory.mktemp("gen_a"), TINY_A, seed=3, storage="float32", loud=True)
    return folder, plain.load_model(folder)


@pytest.fixture(scope="module")
def model_b(tmp_path_factory):
    folder = make_folder(tmp_path_factory.mktemp("gen_b"), TINY_B, seed=4, storage="bfloat16", loud=True)
    return folder, plain.load_model(folder)


def test_greedy_generation_matches_the_plain_implementation(model_a):
    folder, (pcfg, pw) = model_a
    prompts = random_prompts(TINY_A, [5, 9, 17], seed=1)           # the workload of the first tiny configuration
    loaded = AutoCausalLm.load_local(folder, AutoLoadOptions(dtype="float32", max_tokens=64 * 3))
    out = generate_causal(loaded.model, CausalGenerationRequest(prompts, GenerationConfig(max_new_tokens=8)))
    for prompt, seq in zip(prompts, out.sequences):
        want, want_lp = plain.generate(pcfg, pw, prompt, 8)
        assert seq.token_ids == want and seq.prompt_length == len(prompt) and seq.finish_reason.kind == "length"
        assert np.abs(np.array(seq.log_probabilities) - np.array(want_lp)).max() < 1e-3
    assert loaded.model.cache.slots.held == 0


def test_seeded_sampling_is_reproducible_and_does_not_depend_on_the_batch(model_a):
    folder, (pcfg, pw) = model_a
    prompts = random_prompts(TINY_A, [5, 9, 17], seed=2)
    cfg = GenerationConfig(max_new_tokens=8, strategy="sample", temperature=0.8, seed=77)
    loaded = AutoCausalLm.load_local(folder, AutoLoadOptions(dtype="float32", max_tokens=64 * 3))
    together = generate_causal(loaded.model, CausalGenerationRequest(prompts, cfg)).sequences
    again = generate_causal(loaded.model, CausalGenerationRequest(prompts, cfg)).sequences
    one_by_one = generate_causal(loaded.model, CausalGenerationRequest(prompts, cfg, max_batch=1)).sequences
    assert [s.token_ids for s in together] == [s.token_ids for s in again] == [s.token_ids for s in one_by_one]
    other = generate_causal(loaded.model, CausalGenerationRequest(
        prompts, GenerationConfig(max_new_tokens=8, strategy="sample", temperature=0.8, seed=78))).sequences
    assert [s.token_ids for s in other] != [s.token_ids for s in together]
    # (the fourth run of the same prompt shape replays a recorded step: its tokens are checked like the first's)
    for seed, run in ((77, together), (78, other)):
        for r, (prompt, seq) in enumerate(zip(prompts, run)):
            want, _ = plain.generate(pcfg, pw, prompt, 8, sample=True, temperature=0.8, stream=sequence_stream(seed, r))
            assert seq.token_ids == want, (seed, r)


def test_stops_and_streaming_in_bfloat16(model_b):
    folder, (pcfg, pw) = model_b
    prompts = random_prompts(TINY_B, [1, 7, 31, 64], seed=3)       # the workload of the second tiny configuration
    loaded = AutoCausalLm.load_local(folder, AutoLoadOptions(dtype="bfloat16", max_tokens=64 * 6))
    free_run = generate_causal(loaded.model, CausalGenerationRequest(prompts, GenerationConfig(max_new_tokens=12)))
    assert all(len(s.token_ids) == 12 for s in free_run.sequences)
    eos = free_run.sequences[1].token_ids[3]                      # make the second request end early
    seen = []
    out = generate_causal_streaming(loaded.model, CausalGenerationRequest(
        prompts, GenerationConfig(max_new_tokens=12, eos_token_ids=[eos])), seen.append)
    second = out.sequences[1]
    first_hit = free_run.sequences[1].token_ids.index(eos)
    assert second.token_ids == free_run.sequences[1].token_ids[:first_hit + 1]
    assert second.finish_reason.kind == "end_of_sequence" and second.finish_reason.token_id == eos
    for a, b in zip(out.sequences, free_run.sequences):            # the others are not disturbed by the early end
        n = len(a.token_ids)
        assert a.token_ids == b.token_ids[:n]
    assert len(seen) == sum(len(s.token_ids) for s in out.sequences)
    assert loaded.model.cache.slots.held == 0


def test_more_requests_than_the_cache_holds_at_once(model_a):
    folder, (pcfg, pw) = model_a
    prompts = random_prompts(TINY_A, [5, 9, 17, 30, 3, 12, 8], seed=4)
    loaded = AutoCausalLm.load_local(folder, AutoLoadOptions(dtype="float32", max_tokens=64 * 2, max_slots=2))
    out = generate_causal(loaded.model, CausalGenerationRequest(prompts, GenerationConfig(max_new_tokens=6)))
    for prompt, seq in zip(prompts, out.sequences):
        assert seq.token_ids == plain.generate(pcfg, pw, prompt, 6)[0]


def test_penalties_and_filters_change_what_is_generated(model_a):
    folder, (pcfg, pw) = model_a
    prompt = random_prompts(TINY_A, [9], seed=5)
    loaded = AutoCausalLm.load_local(folder, AutoLoadOptions(dtype="float32", max_tokens=64))
    base = generate_causal(loaded.model, CausalGenerationRequest(prompt, GenerationConfig(max_new_tokens=10)))
    banned = base.sequences[0].token_ids[0]
    out = generate_causal(loaded.model, CausalGenerationRequest(
        prompt, GenerationConfig(max_new_tokens=10, logit_bias={banned: -1e4}))).sequences[0]
    assert banned not in out.token_ids
    out = generate_causal(loaded.model, CausalGenerationRequest(
        prompt, GenerationConfig(max_new_tokens=10, no_repeat_ngram_size=1))).sequences[0]
    assert len(set(out.token_ids)) == 10 and not set(out.token_ids) & set(prompt[0])
    # top_k = 1 makes sampling greedy
    out = generate_causal(loaded.model, CausalGenerationRequest(
        prompt, GenerationConfig(max_new_tokens=10, strategy="sample", temperature=1.3, top_k=1, seed=5))).sequences[0]
    assert out.token_ids == base.sequences[0].token_ids


def test_command_line(model_a):
    folder, (pcfg, pw) = model_a
    prompts = random_prompts(TINY_A, [4, 6], seed=6)
    text = ";".join(",".join(map(str, p)) for p in prompts)
    done = subprocess.run([sys.executable, str(ROOT / "bin" / "generate"), str(folder), text, "5", "--dtype", "float32",
                           "--json"], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr
    lines = [json.loads(l) for l in done.stdout.strip().splitlines()]
    assert [l["token_ids"] for l in lines] == [plain.generate(pcfg, pw, p, 5)[0] for p in prompts]
    bad = subprocess.run([sys.executable, str(ROOT / "bin" / "generate"), str(folder), "1,2", "0"], capture_output=True,
                         text=True, timeout=600)
    assert bad.returncode == 2 and "usage" in bad.stderr


@pytest.mark.parametrize("dtype, tol", [("float32", 1e-4), ("bfloat16", 3e-2)])
def test_trace_run_program(model_b, tmp_path, dtype, tol):
    """The replay program fed a trace on standard input: two batches one after another, unequal lengths, the
    shorter requests end earlier, logits wanted at some places only."""
    folder, (pcfg, pw) = model_b
    seqs = dict(zip("abcd", random_prompts(TINY_B, [40, 7, 66, 3], seed=7)))
    steps, expect = [], {}
    n = 0
    for batch, cut in ((("a", "b"), {"a": 33, "b": 1}), (("c", "d"), {"c": 64, "d": 2})):
        steps.append({"step": n, "entries": [{"id": r, "tokens": seqs[r][:cut[r]], "want": [0, cut[r] - 1]} for r in batch],
                      "end": []})
        expect[n] = [(r, p) for r in batch for p in (0, cut[r] - 1)]
        n += 1
        fed = dict(cut)
        while any(fed[r] < len(seqs[r]) for r in batch):
            live = [r for r in batch if fed[r] < len(seqs[r])]
            ends = [r for r in live if fed[r] + 1 == len(seqs[r])]
            wants = [[0] if (fed[r] % 3 == 0 or r in ends) else [] for r in live]
            steps.append({"step": n, "entries": [{"id": r, "tokens": [seqs[r][fed[r]]], "want": w}
                                                 for r, w in zip(live, wants)], "end": ends})
            if any(wants):
                expect[n] = [(r, fed[r]) for r, w in zip(live, wants) if w]
            n += 1
            for r in live:
                fed[r] += 1
    out = tmp_path / "out"
    env = dict(os.environ)
    done = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out),
                           "--max-tokens", str(64 * 3)], input="\n".join(json.dumps(s) for s in steps) + "\n",
                          capture_output=True, text=True, timeout=900, env=env)
    assert done.returncode == 0, done.stderr
    assert done.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    rounded = {k: (plain.round_to_bf16(v) if v.ndim == 2 else v) for k, v in pw.items()}
    quant = plain.round_to_bf16 if dtype == "bfloat16" else None
    ref = {r: plain.logits(pcfg, rounded if quant else pw, s, quant=quant) for r, s in seqs.items()}
    assert sorted(int(p.stem) for p in out.glob("*.f32")) == sorted(expect)
    for step, places in expect.items():
        got = np.frombuffer((out / f"{step}.f32").read_bytes(), dtype="<f4").reshape(len(places), TINY_B["vocab_size"])
        for row, (r, p) in zip(got, places):
            assert np.abs(row - ref[r][p]).max() / np.abs(ref[r]).max() < tol, (step, r, p)


def test_a_reported_wait_that_ran_out_becomes_an_error(model_a):
    """Kernels give up a wait of their own after a limit and say so in a status word; the engine turns that into an
    error where the host waits anyway.  (The report is made here by hand: no kernel is made to wait.)"""
    from burn_transformers_b200 import Engine, KernelError, kernels
    engine = Engine.from_folder(model_a[0], "bfloat16", max_tokens=128)
    engine.check_kernels()
    kernels.kernel_status(engine.device).fill_(3)
    with pytest.raises(KernelError, match="fused decode step"):
        engine.check_kernels()
    engine.check_kernels()          # the report is cleared
