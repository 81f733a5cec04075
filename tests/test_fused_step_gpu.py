"""The fused decode step (one persistent kernel for a whole step) at head sizes, batch sizes and context lengths
that the tiny configurations of the other tests do not reach: against the plain implementation, and its token
selection against the selection kernel on the step's own logits."""
import numpy as np
import pytest
import torch

import engine_replay as replay
import plain_gpt2 as plain
import burn_transformers_b200 as bt
from burn_transformers_b200 import Engine, StepEntry, kernels
from burn_transformers_b200.engine import program as step_program
from burn_transformers_b200.engine.graphs import DecodeSession
from burn_transformers_b200.sampling.sampler import DeviceSampler
from burn_transformers_b200.sampling.tracker import SequenceTracker
from tiny_configs import make_folder, random_prompts

pytestmark = pytest.mark.gpu

TOL_BF16 = 3e-2        # as in test_model_gpu.py: against the plain implementation that rounds where the engine does

# head sizes 64, 96 and 128 (two, three and four 32-wide blocks of a head), widths that are no power of two
FUSED_CONFIGS = {
    "h64": dict(model_type="gpt2", n_layer=2, n_embd=192, n_head=3, n_inner=320, vocab_size=1003, n_positions=704,
                layer_norm_epsilon=1e-5, activation_function="gelu_new"),
    "h96": dict(model_type="gpt2", n_layer=2, n_embd=192, n_head=2, n_inner=256, vocab_size=777, n_positions=704,
                layer_norm_epsilon=2e-5, activation_function="gelu", scale_attn_by_inverse_layer_idx=True),
    "h128": dict(model_type="gpt2", n_layer=1, n_embd=256, n_head=2, n_inner=512, vocab_size=520, n_positions=704,
                 layer_norm_epsilon=1e-5, activation_function="gelu_new"),
}
LENGTHS = [40, 130, 333, 700]


@pytest.fixture(scope="module", params=sorted(FUSED_CONFIGS))
def case(request, tmp_path_factory):
    cfg = FUSED_CONFIGS[request.param]
    folder = make_folder(tmp_path_factory.mktemp(f"fused_{request.param}"), cfg, seed=3, storage="bfloat16", loud=False)
    pcfg, pw = plain.load_model(folder)
    seqs = random_prompts(cfg, LENGTHS, seed=9)
    rounded = {k: (plain.round_to_bf16(v) if v.ndim == 2 else v) for k, v in pw.items()}
    ref = [plain.logits(pcfg, rounded, s, quant=plain.round_to_bf16) for s in seqs]
    return cfg, folder, seqs, ref


def fused_programs(engine):
    return [g.program for g in engine._graphs.values() if g.program is not None]


@pytest.mark.parametrize("splits", [None, 1, 3])
def test_decoding_one_by_one_through_the_fused_step(case, splits, monkeypatch):
    """The last 32 tokens of every request come one at a time: each is one fused step with one sequence.  With one
    split a block takes all pages of a head, more than its ring of page slots holds at once for the long
    requests."""
    cfg, folder, seqs, ref = case
    monkeypatch.setattr(step_program, "SPLITS_OVERRIDE", splits)
    engine = Engine.from_folder(folder, "bfloat16", max_tokens=64 * 12)
    got = replay.tail_one_by_one(engine, seqs)
    assert fused_programs(engine), "the decode steps did not run as a fused step"
    err, where = replay.worst_error(got, ref)
    assert err < TOL_BF16, f"fused tail: {err:.3e} at {where}"


def test_batches_through_the_fused_step(case):
    """Unequal requests decode together (each prompt cut to a third): the steps bring one token per sequence and
    the shorter requests end earlier, so several batch sizes run as fused steps."""
    cfg, folder, seqs, ref = case
    engine = Engine.from_folder(folder, "bfloat16", max_tokens=64 * 24)
    short = [s[:160] for s in seqs] + [s[5:90] for s in seqs]
    pcfg, pw = plain.load_model(folder)
    rounded = {k: (plain.round_to_bf16(v) if v.ndim == 2 else v) for k, v in pw.items()}
    refs = [plain.logits(pcfg, rounded, s, quant=plain.round_to_bf16) for s in short]
    groups = [list(range(len(short)))]
    got = replay.batches(engine, short, groups, [max(1, len(s) // 3) for s in short])
    assert len(fused_programs(engine)) >= 2
    err, where = replay.worst_error(got, refs)
    assert err < TOL_BF16, f"fused batches: {err:.3e} at {where}"


@pytest.mark.parametrize("mode", ["greedy", "sample"])
@pytest.mark.parametrize("batch", [1, 5, 16])
def test_selection_inside_the_fused_step(case, mode, batch):
    """The step's ids and log-probabilities are what the selection kernel gives on the step's own logits, and the
    step moves every sequence on by one token."""
    cfg, folder, seqs, _ = case
    config = bt.GenerationConfig(max_new_tokens=8, strategy=mode, temperature=0.8, top_k=50, top_p=0.9, seed=4)
    engine = Engine.from_folder(folder, "bfloat16", max_tokens=64 * 12 * 16, max_slots=16)
    vocab = cfg["vocab_size"]
    prompts = random_prompts(cfg, [17 + 37 * i for i in range(batch)], seed=2)
    sampler = DeviceSampler(config, vocab, engine.device, batch)
    trackers = [SequenceTracker(i, p, config) for i, p in enumerate(prompts)]
    slots = {i: engine.new_sequence() for i in range(batch)}
    logits = engine.step([StepEntry(slots[i], p, [len(p) - 1]) for i, p in enumerate(prompts)])
    ids, lps = sampler.select(logits, trackers)
    for t, a, b in zip(trackers, ids, lps):
        t.push(a, b)
    engine.cache.reserve([(slots[i], len(prompts[i]) + 8) for i in range(batch)])
    session = DecodeSession(engine, config, batch)
    graph = session._compose(trackers, slots)
    for step in range(4):
        meta = graph.meta
        before = {name: meta.view(name)[:batch].clone() for name in ("tokens", "positions", "past_len", "ctx_len", "counters")}
        step_logits = graph.run()          # (the first run is made of separate kernels; the recording serves the later ones)
        assert graph.program is not None, "the session's step does not run as a fused step"
        torch.cuda.synchronize()
        out_ids = meta.out[:batch].clone()
        out_lp = meta.out[batch:2 * batch].view(torch.float32).clone()
        want = torch.zeros(2 * batch, dtype=torch.int32, device=engine.device)
        s = session.selection
        kernels.sample(step_logits, batch, do_sample=s["do_sample"], temperature=s["temperature"], top_k=s["top_k"],
                       top_p=s["top_p"], min_p=s["min_p"], stream_seeds=meta.seeds if s["do_sample"] else None,
                       counters=before["counters"] if s["do_sample"] else None, out_ids=want[:batch],
                       out_logp=want[batch:].view(torch.float32))
        torch.cuda.synchronize()
        assert out_ids.tolist() == want[:batch].tolist(), f"step {step}"
        np.testing.assert_allclose(out_lp.cpu().numpy(), want[batch:].view(torch.float32).cpu().numpy(), rtol=0, atol=2e-5)
        assert meta.view("tokens")[:batch].tolist() == out_ids.tolist()
        for name in ("positions", "past_len", "ctx_len", "counters"):
            assert meta.view(name)[:batch].tolist() == (before[name] + 1).tolist(), name
        for i in range(batch):     # the host's view of the cache follows, as the session does after reading a step
            engine.cache.commit(slots[i], engine.cache.length(slots[i]) + 1)


def test_fused_and_separate_kernels_agree(case):
    """The same decode steps with the fused step switched off give the same logits beyond bfloat16 rounding."""
    cfg, folder, seqs, ref = case
    fused = Engine.from_folder(folder, "bfloat16", max_tokens=64 * 12)
    plain_path = Engine.from_folder(folder, "bfloat16", max_tokens=64 * 12)
    plain_path.use_fused_step = False
    a = replay.tail_one_by_one(fused, seqs[1:3], tail=8)
    b = replay.tail_one_by_one(plain_path, seqs[1:3], tail=8)
    assert fused_programs(fused) and not fused_programs(plain_path)
    scale = max(float(np.abs(r).max()) for r in ref)
    drift = max(float(np.abs(a[k] - b[k]).max()) for k in a) / scale
    assert drift < TOL_BF16


def test_a_refused_launch_of_the_fused_step_falls_back_to_separate_kernels(case, monkeypatch):
    """A cooperative launch can be refused (it needs every block resident at once).  The refusal is made here by hand
    (the recorded program's launch raises): the engine goes on with a CUDA graph of separate kernels and gives the
    same logits."""
    from burn_transformers_b200 import KernelError
    cfg, folder, seqs, ref = case
    engine = Engine.from_folder(folder, "bfloat16", max_tokens=64 * 12)

    def refuse(self, trace=None):
        raise KernelError("decode_step: launch failed: too many blocks for a cooperative launch")

    monkeypatch.setattr(step_program.DecodeProgram, "launch", refuse)
    got = replay.tail_one_by_one(engine, seqs[:2], tail=5)
    assert engine.use_fused_step is False and not fused_programs(engine)
    err, where = replay.worst_error(got, ref)
    assert err < TOL_BF16, f"after the refusal: {err:.3e} at {where}"


@pytest.mark.parametrize("splits", [None, 1, 3])
def test_fused_step_at_long_contexts_with_loud_weights(splits, monkeypatch, tmp_path):
    """With weights of the usual scale attention is nearly uniform, and a lost or misplaced page of keys moves the
    logits by less than a bfloat16 rounding.  Loud weights make the softmax pick out single keys anywhere in the
    context: contexts of 333 and 700 tokens (6 and 11 pages, more than a block's ring of page slots holds when one
    block takes a whole head), decoded through the fused step with the splits it chooses, with one and with three."""
    cfg = FUSED_CONFIGS["h64"]
    folder = make_folder(tmp_path, cfg, seed=21, storage="bfloat16", loud=True)
    pcfg, pw = plain.load_model(folder)
    seqs = random_prompts(cfg, [333, 700], seed=6)
    rounded = {k: (plain.round_to_bf16(v) if v.ndim == 2 else v) for k, v in pw.items()}
    ref = [plain.logits(pcfg, rounded, s, quant=plain.round_to_bf16) for s in seqs]
    monkeypatch.setattr(step_program, "SPLITS_OVERRIDE", splits)
    engine = Engine.from_folder(folder, "bfloat16", max_tokens=64 * 20)
    got = replay.tail_one_by_one(engine, seqs, tail=12)
    assert fused_programs(engine), "the decode steps did not run as a fused step"
    err, where = replay.worst_error(got, ref)
    assert err < TOL_BF16, f"fused, loud, splits {splits}: {err:.3e} at {where}"
    # both sequences decoding together (two rows, unequal lengths)
    both = replay.batches(engine, seqs, [[0, 1]], [len(s) - 6 for s in seqs])
    err, where = replay.worst_error(both, ref)
    assert err < TOL_BF16, f"fused batch, loud, splits {splits}: {err:.3e} at {where}"


# ---- another norm inside the fused step: a toy architecture with an RMS norm that is defined here ----

import dataclasses
from typing import ClassVar

from burn_transformers_b200.config import Architecture, ModelConfig, register_architecture, unregister_architecture
from burn_transformers_b200.config.base import field
from burn_transformers_b200.engine import LayerCall, ModelPlan
from burn_transformers_b200.parts import (CausalSelfAttention, DenseFeedForward, LearnedPositions, PreNormBlock, TiedReadout,
                                          TokenEmbedding)
from burn_transformers_b200.parts.base import Norm
from burn_transformers_b200.parts.linear import LazyNorm
from burn_transformers_b200.weights import TensorSpec
from burn_transformers_b200.weights.spec import VECTOR


class ToyRmsNorm(Norm):
    """x / sqrt(mean(x^2) + eps) * weight, written with torch operations.  It names the fused decode step's RMS kind,
    so decode steps of few sequences run as one kernel without this class being known to the library."""
    fused_kind = "rmsnorm"
    has_bias = False

    def __init__(self, width, eps):
        self.width, self.eps = width, eps

    def specs(self):
        return {"weight": TensorSpec((self.width,), VECTOR, ("ones",))}

    def forward(self, ctx, x32, out_dtype, rows=None, n_rows=None, lazy=False):
        n = n_rows if n_rows is not None else ctx.n_tokens
        if lazy and out_dtype == torch.bfloat16 and n <= 16:
            return LazyNorm(self, x32, rows, n)
        return self.apply(ctx, x32, out_dtype, rows, n)

    def apply(self, ctx, x32, out_dtype, rows, n):
        x = x32[:n] if rows is None else x32[rows[:n].long()]
        y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * self.t_weight
        out = ctx.ws.take((n, self.width), out_dtype)
        out[:n] = y.to(out_dtype)
        return out


@dataclasses.dataclass
class ToyRmsConfig(ModelConfig):
    FAMILY: ClassVar[str] = "toy_rms"
    MODEL_TYPES: ClassVar[tuple] = ("toy_rms",)
    model_type: str = field("toy_rms")
    vocab: int = field(300)
    width: int = field(160)
    layers: int = field(2)
    heads: int = field(5)
    max_len: int = field(256)

    def validate(self):
        self._check_model_type(self.model_type)
        self._check_extents(("vocab", "width", "layers", "heads", "max_len"))


def build_toy_rms(config: ToyRmsConfig) -> ModelPlan:
    emb = TokenEmbedding(config.vocab, config.width, 0.5)
    pos = LearnedPositions(config.max_len, config.width, 0.5)
    final = ToyRmsNorm(config.width, 1e-6)
    names = {"embed.weight": (emb, "weight"), "pos.weight": (pos, "weight"), "final.weight": (final, "weight")}
    blocks = []
    for i in range(config.layers):
        n1, n2 = ToyRmsNorm(config.width, 1e-6), ToyRmsNorm(config.width, 1e-6)
        mixer = CausalSelfAttention(config.width, config.heads, config.heads, config.width // config.heads, 0.25, bias=False)
        ffn = DenseFeedForward(config.width, 3 * config.width, "gelu_new", bias=False)
        blocks.append(PreNormBlock(n1, mixer, n2, ffn))
        for part_name, part in (("n1", n1), ("mixer", mixer), ("n2", n2), ("ffn", ffn)):
            for local in part.specs():
                names[f"layers.{i}.{part_name}.{local}"] = (part, local)
    return ModelPlan(config=config, embedding=emb, positions=pos, blocks=blocks,
                     schedule=[LayerCall(i) for i in range(config.layers)], final_norm=final, readout=TiedReadout(emb),
                     names=names, vocab=config.vocab, width=config.width, max_context=config.max_len)


def plain_toy_rms(config, w, seq):
    """The toy model on a whole sequence in float64, written from its definition."""
    s, d, heads = len(seq), config.width, config.heads
    hd = d // heads
    rms = lambda t, p: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-6) * w[p + ".weight"]
    gelu = lambda t: 0.5 * t * (1 + torch.tanh(0.7978845608028654 * (t + 0.044715 * t ** 3)))
    x = w["embed.weight"][seq] + w["pos.weight"][:s]
    hidden = torch.arange(s)[None, :] > torch.arange(s)[:, None]
    for layer in range(config.layers):
        p = f"layers.{layer}."
        proj = rms(x, p + "n1") @ w[p + "mixer.qkv.weight"]
        q, k, v = (proj[:, i * d:(i + 1) * d].view(s, heads, hd) for i in range(3))
        out = torch.zeros(s, heads, hd, dtype=torch.float64)
        for h in range(heads):
            out[:, h] = torch.softmax((q[:, h] @ k[:, h].T * 0.25).masked_fill(hidden, -float("inf")), -1) @ v[:, h]
        x = x + out.reshape(s, d) @ w[p + "mixer.out.weight"]
        x = x + gelu(rms(x, p + "n2") @ w[p + "ffn.up.weight"]) @ w[p + "ffn.down.weight"]
    return rms(x, "final") @ w["embed.weight"].T


def test_a_toy_architecture_with_an_rms_norm_decodes_through_the_fused_step(tmp_path):
    """The norm is defined in this file; it only names the kind of norm the fused step may apply in its place."""
    register_architecture(Architecture("toy_rms", ("toy_rms",), ToyRmsConfig, build_toy_rms), replace=True)
    try:
        config = ToyRmsConfig()
        folder = bt.write_random_model(tmp_path, config, seed=11, storage="bfloat16")
        w = {k: torch.from_numpy(v).double() for k, v in plain.read_safetensors(folder / "model.safetensors").items()}
        rng = np.random.default_rng(4)
        seqs = [rng.integers(0, config.vocab, n).tolist() for n in (90, 33, 140)]
        want = [plain_toy_rms(config, w, s).numpy() for s in seqs]
        results = {}
        for fused in (True, False):
            engine = Engine.from_folder(folder, "bfloat16", max_tokens=64 * 8)
            engine.use_fused_step = fused
            results[fused] = replay.tail_one_by_one(engine, seqs, tail=24)
            assert bool(fused_programs(engine)) == fused, "the fused step ran (or did not) against the switch"
        # the fused step against the same model as separate kernels (bfloat16 both, rounding in the same places) ...
        separate = {r: np.stack([results[False][(r, p)] for p in range(len(s))]) for r, s in enumerate(seqs)}
        err, where = replay.worst_error(results[True], separate)
        assert err < TOL_BF16, f"rms norm, fused against separate kernels: {err:.3e} at {where}"
        # ... and both against the model in 64-bit (which rounds nothing): the direction of every row of logits
        for fused, got in results.items():
            for (r, p), row in got.items():
                ref = want[r][p]
                cosine = float(row @ ref / (np.linalg.norm(row) * np.linalg.norm(ref)))
                assert cosine > 0.999, f"rms norm, fused={fused}: cosine {cosine:.5f} at {(r, p)}"
    finally:
        unregister_architecture("toy_rms")
