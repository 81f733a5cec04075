"""Each part alone, and a toy architecture with a stateful mixer that is defined here, registered, built from a
model folder and stepped without touching the library's files."""
import dataclasses
import math
from typing import ClassVar

import numpy as np
import pytest
import torch

import burn_transformers_b200 as bt
from burn_transformers_b200.cache import CacheBank, CacheConfig, CacheNeed, StateSpec
from burn_transformers_b200.config import Architecture, ModelConfig, register_architecture, unregister_architecture
from burn_transformers_b200.config.base import field
from burn_transformers_b200.engine import LayerCall, ModelPlan, StepBuilder, StepEntry
from burn_transformers_b200.parts import (CausalSelfAttention, DenseFeedForward, FeedForward, LayerNorm, LearnedPositions, Mixer,
                                          PositionEncoding,
                                          PreNormBlock, TiedReadout, TokenEmbedding)
from burn_transformers_b200.weights import MATRIX, TensorSpec, random_tensors
from burn_transformers_b200.weights.spec import WeightPlan

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def bound(part, dtype, seed=3):
    """The part with loud random tensors on the device; returns float64 copies of them too."""
    plan = WeightPlan(dict(part.specs()))
    host = random_tensors(plan, seed, storage="bfloat16" if dtype == torch.bfloat16 else "float32", loud=True)
    keep = {n: (t.to(dtype) if plan.tensors[n].kind == MATRIX else t.float()).to(DEV) for n, t in host.items()}
    part.bind(keep)
    return {n: t.double().cpu() for n, t in keep.items()}


def context(needs, entries_tokens, dtype, pasts=None):
    cache = CacheBank(needs, CacheConfig(64 * 16, 8, 512), dtype, DEV)
    builder = StepBuilder(cache, dtype, DEV)
    slots = [cache.acquire() for _ in entries_tokens]
    return cache, builder, slots


TOL = {torch.float32: 1e-5, torch.bfloat16: 1.5e-2}


def rel(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).abs().max() / want.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_and_feed_forward_parts(dtype):
    width, inner, n = 72, 200, 11
    cache, builder, slots = context([], [[0] * n], dtype)
    ctx = builder.build([StepEntry(slots[0], [0] * n, [])])
    norm = LayerNorm(width, 1e-4)
    w = bound(norm, dtype)
    x = torch.randn(n, width, device=DEV) * 2 + 1
    got = norm.forward(ctx, x, dtype)
    want = torch.nn.functional.layer_norm(x.double().cpu(), (width,), w["weight"], w["bias"], 1e-4)
    assert rel(got, want) < TOL[dtype]
    for act, fn in (("gelu_new", lambda t: torch.nn.functional.gelu(t, approximate="tanh")),
                    ("gelu", torch.nn.functional.gelu)):
        ffn = DenseFeedForward(width, inner, act)
        w = bound(ffn, dtype)
        a = torch.randn(n, width, device=DEV).to(dtype)
        residual = torch.randn(n, width, device=DEV)
        want = residual.double().cpu() + fn(a.double().cpu() @ w["up.weight"] + w["up.bias"]) @ w["down.weight"] \
            + w["down.bias"]
        ffn.forward(ctx, a, residual)
        assert rel(residual, want) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_positions_and_readout_parts(dtype):
    vocab, width, n_pos = 300, 40, 50
    emb, pos = TokenEmbedding(vocab, width), LearnedPositions(n_pos, width)
    we, wp = bound(emb, dtype, 1), bound(pos, dtype, 2)
    cache, builder, slots = context([], [[0]], dtype)
    toks = [5, 299, 0, 17]
    ctx = builder.build([StepEntry(slots[0], toks, [3, 0])])
    out = torch.empty(4, width, device=DEV)
    emb.forward(ctx, pos, out)
    assert rel(out, we["weight"][toks] + wp["weight"][:4]) < 1e-6
    h = torch.randn(2, width, device=DEV).to(dtype)
    logits = TiedReadout(emb).forward(ctx, h, 2)
    assert logits.dtype == torch.float32 and rel(logits, h.double().cpu() @ we["weight"].T) < 1e-5


def plain_attention_part(x, w, hq, hkv, hd, scale, window):
    """Whole-sequence attention of one sequence in float64: x [S, width] -> mixer output [S, width]."""
    proj = x @ w["qkv.weight"] + w["qkv.bias"]
    s = x.shape[0]
    q = proj[:, :hq * hd].view(s, hq, hd)
    k = proj[:, hq * hd:(hq + hkv) * hd].view(s, hkv, hd)
    v = proj[:, (hq + hkv) * hd:].view(s, hkv, hd)
    out = torch.zeros(s, hq, hd, dtype=torch.float64)
    i, j = torch.arange(s)[:, None], torch.arange(s)[None, :]
    hidden = j > i
    if window:
        hidden = hidden | (j <= i - window)
    for h in range(hq):
        sc = (q[:, h] @ k[:, h // (hq // hkv)].T * scale).masked_fill(hidden, -math.inf)
        out[:, h] = torch.softmax(sc, -1) @ v[:, h // (hq // hkv)]
    return out.reshape(s, hq * hd) @ w["out.weight"] + w["out.bias"]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hq, hkv, hd, window", [(4, 4, 16, None), (6, 2, 48, None), (2, 1, 32, 20)])
def test_attention_part_prefill_then_decode(dtype, hq, hkv, hd, window):
    """The mixer alone: a prompt in one step and then single tokens give what the whole sequence gives."""
    width, total, prompt = 56, 90, 70
    att = CausalSelfAttention(width, hq, hkv, hd, 0.21, window=window)
    w = bound(att, dtype)
    x = (torch.randn(total, width) * 0.7).to(dtype)
    want = plain_attention_part(x.double(), w, hq, hkv, hd, 0.21, window)
    cache, builder, slots = context([att.cache_need()], [[0]], dtype)
    got = torch.zeros(total, width, dtype=torch.float64)
    steps = [(0, prompt)] + [(p, p + 1) for p in range(prompt, total)]
    for lo, hi in steps:
        entry = StepEntry(slots[0], [0] * (hi - lo), [])
        cache.reserve([(slots[0], hi)])
        ctx = builder.build([entry])
        builder.ws.reset()
        residual = torch.zeros(hi - lo, width, device=DEV)
        att.forward(ctx, x[lo:hi].to(DEV).contiguous(), residual, 0)
        cache.commit(slots[0], hi)
        got[lo:hi] = residual.double().cpu()
    assert rel(got, want) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_part(dtype):
    width = 48
    att = CausalSelfAttention(width, 3, 3, 16, 0.25)
    ffn = DenseFeedForward(width, 100, "gelu_new")
    n1, n2 = LayerNorm(width, 1e-5), LayerNorm(width, 1e-5)
    block = PreNormBlock(n1, att, n2, ffn)
    wa, wf, w1, w2 = bound(att, dtype, 1), bound(ffn, dtype, 2), bound(n1, dtype, 3), bound(n2, dtype, 4)
    n = 33
    x = torch.randn(n, width)
    ln = lambda t, w: torch.nn.functional.layer_norm(t, (width,), w["weight"], w["bias"], 1e-5)
    y = x.double() + plain_attention_part(ln(x.double(), w1), wa, 3, 3, 16, 0.25, None)
    want = y + torch.nn.functional.gelu(ln(y, w2) @ wf["up.weight"] + wf["up.bias"], approximate="tanh") \
        @ wf["down.weight"] + wf["down.bias"]
    cache, builder, slots = context([block.cache_need()], [[0]], dtype)
    cache.reserve([(slots[0], n)])
    ctx = builder.build([StepEntry(slots[0], [0] * n, [])])
    residual = x.to(DEV).clone()
    block.forward(ctx, residual, 0)
    assert rel(residual, want) < (1e-5 if dtype == torch.float32 else 3e-2)


# ---- a toy architecture, defined in this test ---------------------------------------------------------

class RunningMeanMixer(Mixer):
    """Adds `proj @ mean(x[0..t])` to the stream: the mean over everything the sequence has seen so far.
    Its memory is a state of fixed size per sequence (the running sum and the count), not keys per position."""
    graph_safe = False          # written with torch operations, for the test only

    def __init__(self, width):
        self.width = width

    def specs(self):
        return {"proj.weight": TensorSpec((self.width, self.width), MATRIX, ("normal", 0.3))}

    def cache_need(self):
        return CacheNeed(states=(StateSpec("sum", (self.width,)), StateSpec("count", (1,))))

    def forward(self, ctx, x, residual, entry, owns_cache=True):
        total, count = ctx.cache.state(entry, "sum"), ctx.cache.state(entry, "count")
        for i, slot in enumerate(ctx.host_slots):
            lo, hi = ctx.host_seq_start[i], ctx.host_seq_start[i + 1]
            running = total[slot] + torch.cumsum(x[lo:hi].float(), dim=0)
            counts = count[slot] + torch.arange(1, hi - lo + 1, device=x.device, dtype=torch.float32)[:, None]
            residual[lo:hi] += (running / counts) @ self.t_proj_weight.float()
            total[slot] = running[-1]
            count[slot] = counts[-1]


@dataclasses.dataclass
class ToyConfig(ModelConfig):
    FAMILY: ClassVar[str] = "toy_running_mean"
    MODEL_TYPES: ClassVar[tuple] = ("toy_running_mean",)
    model_type: str = field("toy_running_mean")
    vocab: int = field(50)
    width: int = field(32)
    layers: int = field(2)
    heads: int = field(2)
    max_len: int = field(128)

    def validate(self):
        self._check_model_type(self.model_type)
        self._check_extents(("vocab", "width", "layers", "heads", "max_len"))


def build_toy(config: ToyConfig) -> ModelPlan:
    """Layer 0: the stateful toy mixer.  Layer 1: attention.  The run order names layer 0 twice, and the last
    call reads the cache of the attention call before it."""
    emb = TokenEmbedding(config.vocab, config.width, 0.5)
    pos = LearnedPositions(config.max_len, config.width, 0.5)
    final = LayerNorm(config.width, 1e-5)
    names = {"embed.weight": (emb, "weight"), "pos.weight": (pos, "weight"), "final.weight": (final, "weight"),
             "final.bias": (final, "bias")}
    blocks = []
    for i in range(config.layers):
        mixer = RunningMeanMixer(config.width) if i % 2 == 0 else \
            CausalSelfAttention(config.width, config.heads, config.heads, config.width // config.heads, 0.3, bias=False)
        n1, n2 = LayerNorm(config.width, 1e-5), LayerNorm(config.width, 1e-5)
        ffn = DenseFeedForward(config.width, 2 * config.width, "gelu", bias=False)
        blocks.append(PreNormBlock(n1, mixer, n2, ffn))
        for part_name, part in (("n1", n1), ("mixer", mixer), ("n2", n2), ("ffn", ffn)):
            for local in part.specs():
                names[f"layers.{i}.{part_name}.{local}"] = (part, local)
    schedule = [LayerCall(0), LayerCall(1), LayerCall(0), LayerCall(1, cache=1)]
    return ModelPlan(config=config, embedding=emb, positions=pos, blocks=blocks, schedule=schedule, final_norm=final,
                     readout=TiedReadout(emb), names=names, vocab=config.vocab, width=config.width,
                     max_context=config.max_len)


def plain_toy(config, w, seq):
    """The toy model on a whole sequence in float64, written from its definition."""
    s, d, heads = len(seq), config.width, config.heads
    ln = lambda t, p: torch.nn.functional.layer_norm(t, (d,), w[p + ".weight"], w[p + ".bias"], 1e-5)
    x = w["embed.weight"][seq] + w["pos.weight"][:s]
    kv_of_call = {}
    for call, (layer, reads) in enumerate([(0, None), (1, None), (0, None), (1, 1)]):
        p = f"layers.{layer}."
        a = ln(x, p + "n1")
        if layer % 2 == 0:
            mean = torch.cumsum(a, 0) / torch.arange(1, s + 1, dtype=torch.float64)[:, None]
            x = x + mean @ w[p + "mixer.proj.weight"]
        else:
            proj = a @ w[p + "mixer.qkv.weight"]
            hd = d // heads
            q = proj[:, :d].view(s, heads, hd)
            if reads is None:
                kv_of_call[call] = (proj[:, d:2 * d].view(s, heads, hd), proj[:, 2 * d:].view(s, heads, hd))
            k, v = kv_of_call[call if reads is None else reads]
            out = torch.zeros(s, heads, hd, dtype=torch.float64)
            hidden = torch.arange(s)[None, :] > torch.arange(s)[:, None]
            for h in range(heads):
                out[:, h] = torch.softmax((q[:, h] @ k[:, h].T * 0.3).masked_fill(hidden, -math.inf), -1) @ v[:, h]
            x = x + out.reshape(s, d) @ w[p + "mixer.out.weight"]
        f = ln(x, p + "n2")
        x = x + torch.nn.functional.gelu(f @ w[p + "ffn.up.weight"]) @ w[p + "ffn.down.weight"]
    return ln(x, "final") @ w["embed.weight"].T


def test_toy_architecture_with_a_stateful_mixer(tmp_path):
    register_architecture(Architecture("toy_running_mean", ("toy_running_mean",), ToyConfig, build_toy), replace=True)
    try:
        config = ToyConfig()
        folder = bt.write_random_model(tmp_path, config, seed=5, storage="float32")
        engine = bt.Engine.from_folder(folder, "float32", max_tokens=64 * 6)
        assert not engine.plan.graph_safe
        assert len(engine.cache.groups) == 1 and engine.cache.groups[0].k.shape[0] == 1    # one owner of keys
        import plain_gpt2
        w = {k: torch.from_numpy(v) for k, v in plain_gpt2.read_safetensors(folder / "model.safetensors").items()}
        rng = np.random.default_rng(0)
        seqs = [rng.integers(0, 50, n).tolist() for n in (70, 9, 33)]
        want = [plain_toy(config, w, s) for s in seqs]
        for round_ in range(2):                       # the second round reuses slots whose state must be zero again
            slots = [engine.new_sequence() for _ in seqs]
            cut = [20, 1, 33]
            got = engine.step([StepEntry(sl, s[:c], list(range(c))) for sl, s, c in zip(slots, seqs, cut)])
            off = 0
            for r, c in enumerate(cut):
                assert rel(got[off:off + c], want[r][:c]) < 1e-4
                off += c
            fed = list(cut)
            while any(f < len(s) for f, s in zip(fed, seqs)):
                live = [r for r in range(3) if fed[r] < len(seqs[r])]
                got = engine.step([StepEntry(slots[r], [seqs[r][fed[r]]], [0]) for r in live])
                for i, r in enumerate(live):
                    assert rel(got[i], want[r][fed[r]]) < 1e-4, (round_, r, fed[r])
                    fed[r] += 1
            for sl in slots:
                engine.release(sl)
            engine.cache.check()
    finally:
        unregister_architecture("toy_running_mean")


# ---- a second toy architecture: a position encoding that rotates, a windowed layer, a routed feed-forward ----

class ToyRotation(PositionEncoding):
    """Rotates pairs (2i, 2i + 1) of every query and key head by position * base^(-2i / head_dim); angles in
    32-bit.  Defined here with torch operations: the framework only knows the `rotate` hook."""
    rotates = True
    graph_safe = False

    def __init__(self, base: float):
        self.base = base

    def rotate(self, ctx, proj, n_heads, n_kv_heads, head_dim):
        n = ctx.n_tokens
        pos = ctx.positions[:n].to(torch.float32)
        freq = self.base ** (-torch.arange(0, head_dim, 2, device=proj.device, dtype=torch.float32) / head_dim)
        angle = pos[:, None] * freq[None, :]
        cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
        heads = proj[:n, :(n_heads + n_kv_heads) * head_dim].view(n, n_heads + n_kv_heads, head_dim // 2, 2).to(torch.float32)
        a, b = heads[..., 0], heads[..., 1]
        turned = torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1)
        proj[:n, :(n_heads + n_kv_heads) * head_dim] = turned.reshape(n, -1).to(proj.dtype)


class ToyRoutedFeedForward(FeedForward):
    """Every token goes to the one expert its router logit (32-bit) is largest for; an expert is up, GELU, down."""
    graph_safe = False

    def __init__(self, width, inner, experts):
        self.width, self.inner, self.experts = width, inner, experts

    def specs(self):
        specs = {"router.weight": TensorSpec((self.width, self.experts), MATRIX, ("normal", 1.0))}
        for e in range(self.experts):
            specs[f"experts.{e}.up.weight"] = TensorSpec((self.width, self.inner), MATRIX, ("normal", 0.3))
            specs[f"experts.{e}.down.weight"] = TensorSpec((self.inner, self.width), MATRIX, ("normal", 0.3))
        return specs

    def forward(self, ctx, x, residual):
        n = ctx.n_tokens
        rows = x[:n].float()
        choice = (rows @ self.t_router_weight.float()).argmax(dim=1)
        for e in range(self.experts):
            mine = (choice == e).nonzero().flatten()
            if mine.numel():
                hidden = torch.nn.functional.gelu(rows[mine] @ getattr(self, f"t_experts_{e}_up_weight").float())
                residual[mine] += hidden @ getattr(self, f"t_experts_{e}_down_weight").float()


@dataclasses.dataclass
class RoutedConfig(ModelConfig):
    FAMILY: ClassVar[str] = "toy_routed"
    MODEL_TYPES: ClassVar[tuple] = ("toy_routed",)
    model_type: str = field("toy_routed")
    vocab: int = field(40)
    width: int = field(32)
    heads: int = field(2)
    kv_heads: int = field(1)
    window: int = field(24)
    experts: int = field(3)
    rotary_base: float = field(100.0)
    max_len: int = field(128)

    def validate(self):
        self._check_model_type(self.model_type)
        self._check_extents(("vocab", "width", "heads", "kv_heads", "window", "experts", "max_len"))


def build_routed(config: RoutedConfig) -> ModelPlan:
    """Layer 0: rotated, windowed, grouped-head attention and a routed feed-forward.  Layer 1: plain attention over
    all keys (no rotation) and a dense feed-forward: two groups of cache with different needs."""
    emb = TokenEmbedding(config.vocab, config.width, 0.5)
    rotation = ToyRotation(config.rotary_base)
    final = LayerNorm(config.width, 1e-5)
    hd = config.width // config.heads
    mixers = [CausalSelfAttention(config.width, config.heads, config.kv_heads, hd, 0.3, window=config.window, bias=False,
                                  init_std=0.4, positions=rotation),
              CausalSelfAttention(config.width, config.heads, config.heads, hd, 0.3, bias=False, init_std=0.4)]
    ffns = [ToyRoutedFeedForward(config.width, 2 * config.width, config.experts),
            DenseFeedForward(config.width, 2 * config.width, "gelu", bias=False)]
    names = {"embed.weight": (emb, "weight"), "final.weight": (final, "weight"), "final.bias": (final, "bias")}
    blocks = []
    for i in range(2):
        n1, n2 = LayerNorm(config.width, 1e-5), LayerNorm(config.width, 1e-5)
        blocks.append(PreNormBlock(n1, mixers[i], n2, ffns[i]))
        for part_name, part in (("n1", n1), ("mixer", mixers[i]), ("n2", n2), ("ffn", ffns[i])):
            for local in part.specs():
                names[f"layers.{i}.{part_name}.{local}"] = (part, local)
    return ModelPlan(config=config, embedding=emb, positions=rotation, blocks=blocks, schedule=[LayerCall(0), LayerCall(1)],
                     final_norm=final, readout=TiedReadout(emb), names=names, vocab=config.vocab, width=config.width,
                     max_context=config.max_len)


def plain_routed(config, w, seq):
    """The second toy model on a whole sequence in float64, written from its definition."""
    s, d, heads, kvh = len(seq), config.width, config.heads, config.kv_heads
    hd = d // heads
    ln = lambda t, p: torch.nn.functional.layer_norm(t, (d,), w[p + ".weight"], w[p + ".bias"], 1e-5)
    x = w["embed.weight"][seq]
    pos = torch.arange(s, dtype=torch.float64)
    freq = config.rotary_base ** (-torch.arange(0, hd, 2, dtype=torch.float64) / hd)
    cos, sin = (pos[:, None] * freq).cos()[:, None, :], (pos[:, None] * freq).sin()[:, None, :]

    def turn(t):                       # [s, h, hd]
        a, b = t[..., 0::2], t[..., 1::2]
        return torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1).reshape(t.shape)

    for layer in range(2):
        p = f"layers.{layer}."
        n_kv = kvh if layer == 0 else heads
        proj = ln(x, p + "n1") @ w[p + "mixer.qkv.weight"]
        q = proj[:, :d].view(s, heads, hd)
        k = proj[:, d:d + n_kv * hd].view(s, n_kv, hd)
        v = proj[:, d + n_kv * hd:].view(s, n_kv, hd)
        if layer == 0:
            q, k = turn(q), turn(k)
        hidden = torch.arange(s)[None, :] > torch.arange(s)[:, None]
        if layer == 0:
            hidden |= torch.arange(s)[None, :] <= torch.arange(s)[:, None] - config.window
        out = torch.zeros(s, heads, hd, dtype=torch.float64)
        for h in range(heads):
            kh = h // (heads // n_kv)
            out[:, h] = torch.softmax((q[:, h] @ k[:, kh].T * 0.3).masked_fill(hidden, -math.inf), -1) @ v[:, kh]
        x = x + out.reshape(s, d) @ w[p + "mixer.out.weight"]
        f = ln(x, p + "n2")
        if layer == 0:
            choice = (f @ w[p + "ffn.router.weight"]).argmax(dim=1)
            for e in range(config.experts):
                mine = (choice == e).nonzero().flatten()
                x[mine] = x[mine] + torch.nn.functional.gelu(f[mine] @ w[p + f"ffn.experts.{e}.up.weight"]) \
                    @ w[p + f"ffn.experts.{e}.down.weight"]
        else:
            x = x + torch.nn.functional.gelu(f @ w[p + "ffn.up.weight"]) @ w[p + "ffn.down.weight"]
    return ln(x, "final") @ w["embed.weight"].T


def test_toy_architecture_with_rotation_a_window_and_routed_experts(tmp_path):
    """Parts the library does not have, defined here and registered without a change to its files: a position
    encoding that turns queries and keys, a feed-forward that routes tokens to experts; the model's first layer keeps
    a window of keys (a ring of pages) with shared key heads, its second all keys."""
    register_architecture(Architecture("toy_routed", ("toy_routed",), RoutedConfig, build_routed), replace=True)
    try:
        config = RoutedConfig()
        folder = bt.write_random_model(tmp_path, config, seed=8, storage="float32")
        engine = bt.Engine.from_folder(folder, "float32", max_tokens=64 * 6)
        assert not engine.plan.graph_safe
        assert len(engine.cache.groups) == 2 and sorted(g.is_ring for g in engine.cache.groups) == [False, True]
        import plain_gpt2
        w = {k: torch.from_numpy(v).double() for k, v in plain_gpt2.read_safetensors(folder / "model.safetensors").items()}
        rng = np.random.default_rng(1)
        seqs = [rng.integers(0, config.vocab, n).tolist() for n in (90, 9, 40)]
        want = [plain_routed(config, w, s) for s in seqs]
        for round_ in range(2):
            slots = [engine.new_sequence() for _ in seqs]
            cut = [30, 1, 40]
            got = engine.step([StepEntry(sl, s[:c], list(range(c))) for sl, s, c in zip(slots, seqs, cut)])
            off = 0
            for r, c in enumerate(cut):
                assert rel(got[off:off + c], want[r][:c]) < 1e-4, (round_, r)
                off += c
            fed = list(cut)
            while any(f < len(s) for f, s in zip(fed, seqs)):
                live = [r for r in range(3) if fed[r] < len(seqs[r])]
                got = engine.step([StepEntry(slots[r], [seqs[r][fed[r]]], [0]) for r in live])
                for i, r in enumerate(live):
                    assert rel(got[i], want[r][fed[r]]) < 1e-4, (round_, r, fed[r])
                    fed[r] += 1
            for sl in slots:
                engine.release(sl)
            engine.cache.check()
        # a step may bring several tokens to a sequence that already holds some: as many as the windowed layer's ring
        # of pages allows (64 - 24 + 1 = 41 here); the run 50..79 wraps around the ring
        assert engine.cache.max_continued_run == 41
        slot = engine.new_sequence()
        seq = seqs[0]
        engine.step([StepEntry(slot, seq[:50], [])])
        got = engine.step([StepEntry(slot, seq[50:80], list(range(30)))])
        assert rel(got, want[0][50:80]) < 1e-4
        with pytest.raises(bt.CacheError, match="at most 41 tokens"):
            engine.step([StepEntry(slot, (seq * 2)[:42], [])])
        assert engine.length(slot) == 80
        got = engine.step([StepEntry(slot, seq[80:], [len(seq) - 81])])
        assert rel(got[0], want[0][-1]) < 1e-4
        engine.release(slot)
        with pytest.raises(bt.GenerationError, match="prefill_chunk_size 42"):
            bt.generate(engine, [seq[:50]], bt.GenerationConfig(max_new_tokens=2), prefill_chunk_size=42)
    finally:
        unregister_architecture("toy_routed")


def test_a_checkpoint_with_separate_transposed_projections_runs_in_the_same_parts(tmp_path):
    """Queries, keys and values stored as three [out, in] matrices (and the other projections transposed too) load
    into the unchanged CausalSelfAttention and DenseFeedForward through the plan's sources, and the engine gives
    bit for bit the logits of the fused [in, out] checkpoint."""
    from burn_transformers_b200.weights import load_weights
    from test_weights import split_qkv_plan, store_split
    from tiny_configs import TINY_B, make_folder, random_prompts
    fused = make_folder(tmp_path / "fused", TINY_B, seed=5, storage="float32", loud=True)
    split = make_folder(tmp_path / "split", TINY_B, seed=5, storage="float32", loud=True)
    store_split(split)
    seqs = random_prompts(TINY_B, [19, 70], seed=2)
    for dtype in ("float32", "bfloat16"):
        want_engine = bt.Engine.from_folder(fused, dtype, max_tokens=64 * 4)
        plan = split_qkv_plan(split)
        tensors, _ = load_weights(split, plan.weights, dtype, torch.device(DEV))
        got_engine = bt.Engine(plan, tensors, dtype, CacheConfig(64 * 4, 4, plan.max_context), DEV)
        for seq in seqs:
            logits = []
            for engine in (want_engine, got_engine):
                slot = engine.new_sequence()
                logits.append(engine.step([StepEntry(slot, seq, list(range(len(seq))))]).clone())
                engine.release(slot)
            assert torch.equal(logits[0], logits[1])
