"""The engine against the plain implementation: whole requests, the last 32 tokens one by one, batches of
unequal lengths one after another, long decoding and the first tokens, in 32-bit and in bfloat16."""
import numpy as np
import pytest

import engine_replay as replay
import plain_gpt2 as plain
from burn_transformers_b200 import Engine
from tiny_configs import CONFIGS, make_folder, random_prompts

pytestmark = pytest.mark.gpu

# 32-bit: the target of the whole path, relative to the largest logit of the sequence.
TOL_F32 = 1e-4
# bfloat16: activations are rounded to 8 bits of mantissa (2^-8 = 3.9e-3 per rounding) at about eight places
# per layer, which allows about sqrt(8 * layers) * 3.9e-3.  The bfloat16 engine is compared with the plain
# implementation of the model it serves: matrices rounded to bfloat16 as the loader rounds them, and
# activations rounded where the engine stores them in bfloat16.  (Without that, a configuration whose scores
# are not scaled by 1/sqrt(head size) has softmaxes so sharp that rounding the queries and keys alone moves
# logits by tens of percent: the 32-bit tests cover that configuration's logic.)
TOL_BF16 = 3e-2
LENGTHS = {"A": [5, 9, 17, 40, 70, 101], "B": [1, 7, 31, 64, 65, 130], "C": [3, 64, 90, 129]}


@pytest.fixture(scope="module", params=["A", "B", "C"])
def case(request, tmp_path_factory):
    name = request.param
    cfg = CONFIGS[name]
    storage = {"A": "float32", "B": "bfloat16", "C": "float32"}[name]
    folder = make_folder(tmp_path_factory.mktemp(f"model{name}"), cfg, seed=11, storage=storage, loud=True)
    pcfg, pw = plain.load_model(folder)
    seqs = random_prompts(cfg, LENGTHS[name], seed=5)
    ref = [plain.logits(pcfg, pw, s) for s in seqs]
    rounded = {k: (plain.round_to_bf16(v) if v.ndim == 2 else v) for k, v in pw.items()}
    ref_bf16 = [plain.logits(pcfg, rounded, s, quant=plain.round_to_bf16) for s in seqs]
    return name, cfg, folder, seqs, {"float32": ref, "bfloat16": ref_bf16}


def engine_for(folder, dtype, max_tokens=64 * 12, **kw):
    return Engine.from_folder(folder, dtype, max_tokens=max_tokens, **kw)


@pytest.mark.parametrize("dtype, tol", [("float32", TOL_F32), ("bfloat16", TOL_BF16)])
def test_each_request_whole(case, dtype, tol):
    _, _, folder, seqs, refs = case
    ref = refs[dtype]
    got = replay.whole(engine_for(folder, dtype), seqs)
    assert len(got) == sum(len(s) for s in seqs)
    err, where = replay.worst_error(got, ref)
    assert err < tol, f"whole {dtype}: {err:.3e} at {where}"


@pytest.mark.parametrize("dtype, tol", [("float32", TOL_F32), ("bfloat16", TOL_BF16)])
def test_last_32_tokens_one_by_one(case, dtype, tol):
    _, _, folder, seqs, refs = case
    ref = refs[dtype]
    got = replay.tail_one_by_one(engine_for(folder, dtype), seqs)
    err, where = replay.worst_error(got, ref)
    assert err < tol, f"tail {dtype}: {err:.3e} at {where}"


@pytest.mark.parametrize("dtype, tol", [("float32", TOL_F32), ("bfloat16", TOL_BF16)])
def test_batches_of_unequal_lengths_reuse_slots(case, dtype, tol):
    name, _, folder, seqs, refs = case
    ref = refs[dtype]
    n = len(seqs)
    groups = [list(range(0, n, 2)), list(range(1, n, 2)), list(range(n))[:3]]
    prompt_lengths = [max(1, len(s) // 3) for s in seqs]
    prompt_lengths[0] = 1                      # a request whose first step brings one token among longer ones
    need = max(sum(-(-len(seqs[r]) // 64) * 64 for r in g) for g in groups)
    engine = engine_for(folder, dtype, max_tokens=need)      # exactly what the largest batch needs: pages are reused
    got = replay.batches(engine, seqs, groups, prompt_lengths)
    err, where = replay.worst_error(got, ref)
    assert err < tol, f"batches {dtype}: {err:.3e} at {where}"
    assert engine.cache.slots.held == 0 and all(g.pool.held == 0 for g in engine.cache.groups)
    # the same requests alone give the same logits as in a batch, beyond rounding
    alone = replay.whole(engine, seqs)
    drift = max(float(np.abs(alone[k] - got[k]).max() / np.abs(ref[k[0]]).max()) for k in got)
    assert drift < tol


@pytest.mark.parametrize("dtype, tol", [("float32", TOL_F32), ("bfloat16", TOL_BF16)])
def test_long_decoding_from_the_first_token(case, dtype, tol):
    _, cfg, folder, seqs, refs = case
    ref = refs[dtype]
    long = max(range(len(seqs)), key=lambda r: len(seqs[r]))
    engine = engine_for(folder, dtype)
    got = replay.tail_one_by_one(engine, [seqs[long]], tail=10 ** 6)      # a one-token prompt, then one by one
    err, where = replay.worst_error(got, [ref[long]])
    assert len(got) == len(seqs[long]) and err < tol, f"long decode {dtype}: {err:.3e} at {where}"


def test_padding_free_batch_equals_alone_exactly_in_32_bit(case):
    """In 32-bit every kernel computes a row from that row's data alone, in a fixed order: a request's
    logits are bit-identical alone and in a batch."""
    _, _, folder, seqs, _ = case
    engine = engine_for(folder, "float32")
    alone = replay.whole(engine, seqs[:3])
    together = replay.batches(engine, seqs[:3], [[0, 1, 2]], [len(s) for s in seqs[:3]])
    assert all(np.array_equal(alone[k], together[k]) for k in alone)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_bfloat16_agrees_with_32_bit_on_ordinary_weights(name, tmp_path):
    """With weights of the usual scale the two precisions give the same picture: the logits of a position point the
    same way (cosine >= 0.999, the reference's bound for a reduced-precision run, BENCHMARKS.md:111-112), and the
    most likely token is the same wherever 32-bit leaves no doubt about it."""
    cfg = CONFIGS[name]
    folder = make_folder(tmp_path, cfg, seed=17, storage="float32", loud=False)
    seqs = random_prompts(cfg, [33, 70, 101], seed=4)
    a = replay.whole(engine_for(folder, "float32"), seqs)
    b = replay.whole(engine_for(folder, "bfloat16"), seqs)
    for key in a:
        x, y = a[key].astype(np.float64), b[key].astype(np.float64)
        cosine = float(x @ y / (np.linalg.norm(x) * np.linalg.norm(y)))
        assert cosine >= 0.999, f"{key}: cosine {cosine}"
        top2 = np.sort(x)[-2:]
        if top2[1] - top2[0] > 0.05 * np.abs(x).max():      # 32-bit is decided by a margin far above bfloat16 rounding
            assert int(np.argmax(x)) == int(np.argmax(y)), key
