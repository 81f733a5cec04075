"""Layers of the published GPT-2 sizes (width 1024 / 16 heads, and width 1600 / 25 heads with the full vocabulary), with
few layers and random weights: the kernels meet sizes here that the tiny configurations do not have (a width that is
no power of two, 25 heads, a vocabulary of 50,257, products long enough for every path of the matrix kernels)."""
import numpy as np
import pytest

import engine_replay as replay
import plain_gpt2 as plain
from burn_transformers_b200 import Engine
from tiny_configs import make_folder, random_prompts

pytestmark = pytest.mark.gpu

SIZES = {
    "medium": dict(model_type="gpt2", n_layer=2, n_embd=1024, n_head=16, vocab_size=5003, n_positions=1024),
    "xl": dict(model_type="gpt2", n_layer=1, n_embd=1600, n_head=25, vocab_size=50257, n_positions=1024),
}
LENGTHS = [150, 37, 90]


@pytest.fixture(scope="module", params=sorted(SIZES))
def case(request, tmp_path_factory):
    cfg = SIZES[request.param]
    folder = make_folder(tmp_path_factory.mktemp(f"gpt2_{request.param}"), cfg, seed=21, storage="bfloat16", loud=False)
    pcfg, pw = plain.load_model(folder)
    seqs = random_prompts(cfg, LENGTHS, seed=8)
    rounded = {k: (plain.round_to_bf16(v) if v.ndim == 2 else v) for k, v in pw.items()}
    ref = [plain.logits(pcfg, rounded, s, quant=plain.round_to_bf16) for s in seqs]
    ref32 = [plain.logits(pcfg, pw, seqs[1])]
    return cfg, folder, seqs, ref, ref32


def test_prompts_whole_and_their_tails_one_by_one_in_bfloat16(case):
    cfg, folder, seqs, ref, _ = case
    engine = Engine.from_folder(folder, "bfloat16", max_tokens=64 * 8)
    got = replay.whole(engine, seqs)
    err, where = replay.worst_error(got, ref)
    assert err < 3e-2, f"whole: {err:.3e} at {where}"
    got = replay.tail_one_by_one(engine, seqs, tail=6)
    err, where = replay.worst_error(got, ref)
    assert err < 3e-2, f"tail: {err:.3e} at {where}"
    assert any(g.program is not None for g in engine._graphs.values()), "the decode steps did not run as a fused step"
    engine.use_fused_step = False
    engine._graphs.clear()
    got = replay.tail_one_by_one(engine, seqs, tail=3)
    err, where = replay.worst_error(got, ref)
    assert err < 3e-2, f"tail as separate kernels: {err:.3e} at {where}"


def test_a_batch_of_unequal_requests_in_bfloat16(case):
    cfg, folder, seqs, ref, _ = case
    engine = Engine.from_folder(folder, "bfloat16", max_tokens=64 * 8)
    got = replay.batches(engine, seqs, [[0, 1, 2]], [140, 30, 85])
    err, where = replay.worst_error(got, ref)
    assert err < 3e-2, f"batch: {err:.3e} at {where}"


def test_a_request_in_true_32_bit(case):
    cfg, folder, seqs, _, ref32 = case
    engine = Engine.from_folder(folder, "float32", max_tokens=64 * 2)
    got = replay.tail_one_by_one(engine, [seqs[1]], tail=4)
    err, where = replay.worst_error(got, ref32)
    assert err < 1e-4, f"float32: {err:.3e} at {where}"
