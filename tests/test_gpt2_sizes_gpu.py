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


def test_six_requests_over_wide_layers_decode_as_separate_kernels(case):
    """Six and more rows over layers of 5.5 M weights and more are not recorded as a fused step: the decode steps run
    as a graph of separate kernels (with the tcgen05 product for few rows over the large weights), and give the same
    logits; smaller batches of the same model still take the fused step."""
    cfg, folder, _, _, _ = case
    if cfg["n_embd"] < 1600:
        pytest.skip("the layers of this size stay inside the fused step at every batch")
    pcfg, pw = plain.load_model(folder)
    rounded = {k: (plain.round_to_bf16(v) if v.ndim == 2 else v) for k, v in pw.items()}
    lengths = [20, 35, 50, 28, 41, 33]
    seqs = random_prompts(cfg, lengths, seed=9)
    ref = [plain.logits(pcfg, rounded, s, quant=plain.round_to_bf16) for s in seqs]
    engine = Engine.from_folder(folder, "bfloat16", max_tokens=64 * 6)
    got = replay.batches(engine, seqs, [[0, 1, 2, 3, 4, 5]], [n - 6 for n in lengths])
    err, where = replay.worst_error(got, ref)
    assert err < 3e-2, f"batch of six: {err:.3e} at {where}"
    graphs = {g.n: g for g in engine._graphs.values()}
    assert graphs[6].program is None, "six rows over these layers were recorded as a fused step"
    got = replay.batches(engine, seqs[:3], [[0, 1, 2]], [n - 4 for n in lengths[:3]])
    err, where = replay.worst_error(got, ref[:3])
    assert err < 3e-2, f"batch of three: {err:.3e} at {where}"
    graphs = {g.n: g for g in engine._graphs.values()}
    assert graphs[3].program is not None, "three rows of this model did not run as a fused step"
