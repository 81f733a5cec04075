"""Plain, slow GPT-2 for the tests: whole sequences, no cache, NumPy only.

This file is the oracle of the test suite.  It shares no code with the
package: it has its own safetensors reader, its own configuration reading, its
own sampler.  Every function restates one formula of the reference project
(NoahIsCool/burn-transformers); the citation after each docstring's first line
gives the file and lines, relative to that project's root, that the formula
was read from.

The reference's own model code is Rust on the Burn framework and cannot be
compiled in this environment (no cargo, no rustc), so this file rests on the
formulas.  It is anchored once on the reference's committed PyTorch fixture
(`tests/golden/gpt2_tiny_reference.json`, see `tests/golden/README.md`).

Arithmetic is float64 unless a `quant` callable is given.  `quant` rounds an
array to the storage precision of the engine's reduced-precision path (bfloat16)
at the places where that path stores activations, so that a comparison can be
tighter than the bare bfloat16 error bound.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np

F64 = np.float64


# --------------------------------------------------------------------------
# files
# --------------------------------------------------------------------------

def bf16_bits_to_f32(raw: np.ndarray) -> np.ndarray:
    """uint16 bfloat16 bit patterns -> float32 (exact)."""
    return (raw.astype(np.uint32) << 16).view(np.float32)


def round_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round to nearest-even bfloat16 and return the values as float64."""
    f = np.ascontiguousarray(x, dtype=np.float32)
    bits = f.view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    out = rounded.astype(np.uint32).view(np.float32)
    out = np.where(np.isfinite(f), out, f)
    return out.astype(F64).reshape(np.shape(x))


def read_safetensors(path) -> dict[str, np.ndarray]:
    """Minimal reader: 8-byte little-endian header length, JSON header, raw bytes."""
    blob = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n])
    data = memoryview(blob)[8 + n:]
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = bytes(data[lo:hi])
        dt = meta["dtype"]
        if dt == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(F64)
        elif dt == "BF16":
            arr = bf16_bits_to_f32(np.frombuffer(raw, dtype="<u2")).astype(F64)
        elif dt == "F16":
            arr = np.frombuffer(raw, dtype="<f2").astype(F64)
        else:
            raise ValueError(f"{name}: dtype {dt} not handled by the plain reader")
        out[name] = arr.reshape(meta["shape"])
    return out


def read_config(path) -> dict:
    """config.json with the defaults of GPT-2 small.  (src/models/gpt2.rs:149-171)"""
    cfg = json.loads(Path(path).read_text())
    alias = {"hidden_size": "n_embd", "num_hidden_layers": "n_layer",
             "num_attention_heads": "n_head", "max_position_embeddings": "n_positions"}
    for a, b in alias.items():  # src/models/gpt2.rs:113-123
        if a in cfg and b not in cfg:
            cfg[b] = cfg[a]
    defaults = dict(vocab_size=50257, n_embd=768, n_layer=12, n_head=12, n_positions=1024,
                    n_inner=None, activation_function="gelu_new", layer_norm_epsilon=1e-5,
                    scale_attn_weights=True, scale_attn_by_inverse_layer_idx=False, causal=True)
    for k, v in defaults.items():
        cfg.setdefault(k, v)
    return cfg


def load_model(folder):
    folder = Path(folder)
    cfg = read_config(folder / "config.json")
    w = read_safetensors(folder / "model.safetensors")
    if "transformer.wte.weight" in w:  # src/models/gpt2/checkpoint.rs:46-71
        w = {k[len("transformer."):]: v for k, v in w.items() if k.startswith("transformer.")}
    return cfg, w


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------

def intermediate_width(cfg) -> int:
    """n_inner, or four times the width when absent.  (src/models/gpt2/extents.rs:99-105)"""
    return cfg["n_inner"] if cfg.get("n_inner") else 4 * cfg["n_embd"]


def embed(ids, positions, wte, wpe):
    """x0[t] = wte[id[t]] + wpe[pos[t]].  (src/models/gpt2/model.rs:428-450)"""
    return wte[np.asarray(ids)] + wpe[np.asarray(positions)]


def layer_norm(x, gamma, beta, eps):
    """Biased variance over the last axis, affine.  (src/models/gpt2/model.rs:143-148, 235-239)"""
    mu = x.mean(axis=-1, keepdims=True)
    var = ((x - mu) ** 2).mean(axis=-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * gamma + beta


def conv1d(x, weight, bias):
    """y = x @ W[in,out] + b, no transpose.  (src/models/gpt2/model.rs:95-105, src/operations.rs:529-643)"""
    return x @ weight + bias


def split_heads(x, n_head):
    """[S, H*hd] -> [H, S, hd]; head h owns channels h*hd..(h+1)*hd.  (src/attention.rs:481-486, 528-531)"""
    s, d = x.shape
    return x.reshape(s, n_head, d // n_head).transpose(1, 0, 2)


def merge_heads(x):
    """[H, S, hd] -> [S, H*hd].  (src/attention.rs:882-892)"""
    h, s, hd = x.shape
    return x.transpose(1, 0, 2).reshape(s, h * hd)


def score_scale(cfg, layer: int) -> float:
    """(1/sqrt(hd) if scale_attn_weights) / (layer+1 if scale_attn_by_inverse_layer_idx).
    (src/models/gpt2/model.rs:121-133)"""
    hd = cfg["n_embd"] // cfg["n_head"]
    s = 1.0 / math.sqrt(hd) if cfg["scale_attn_weights"] else 1.0
    if cfg["scale_attn_by_inverse_layer_idx"]:
        s /= (layer + 1)
    return s


def excluded(n_query, n_key, causal=True, key_valid=None, window=None):
    """True where key j is hidden from query i: bottom-right causal
    (j > i + (K-Q)) or padded key.  (src/attention/mask.rs:28-40, 86-107)
    `window` (not used by GPT-2) additionally hides keys more than window-1 behind."""
    i = np.arange(n_query)[:, None] + (n_key - n_query)
    j = np.arange(n_key)[None, :]
    ex = np.zeros((n_query, n_key), dtype=bool)
    if causal:
        ex |= j > i
    if window is not None:
        ex |= j <= i - window
    if key_valid is not None:
        ex |= ~np.asarray(key_valid, dtype=bool)[None, :]
    return ex


def softmax_rows(scores, ex):
    """Excluded scores become -inf; a row with every score excluded is all zeros.
    (src/attention/dispatch.rs:359-406)"""
    s = np.where(ex, -np.inf, scores)
    m = s.max(axis=-1, keepdims=True)
    m = np.where(np.isfinite(m), m, 0.0)
    e = np.exp(s - m)
    z = e.sum(axis=-1, keepdims=True)
    return np.where(z > 0, e / np.where(z > 0, z, 1.0), 0.0)


def attention(q, k, v, scale, causal=True, key_valid=None, window=None, quant=None):
    """softmax((q k^T) * scale) v per head.  (src/attention/dispatch.rs:277-301, 314-328, 420-430)
    q: [H, Q, hd]; k, v: [Hkv, K, hd]; query heads share key heads in consecutive groups
    (GPT-2: Hkv == H)."""
    h, nq, _ = q.shape
    hkv, nk, _ = k.shape
    group = h // hkv
    ex = excluded(nq, nk, causal, key_valid, window)
    out = np.empty_like(q)
    for head in range(h):
        kk, vv = k[head // group], v[head // group]
        p = softmax_rows((q[head] @ kk.T) * scale, ex)
        out[head] = p @ vv
    return out


def gelu_new(x):
    """0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))).  (src/feed_forward.rs:351-406)"""
    return 0.5 * x * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))


def gelu_erf(x):
    """x (1 + erf(x / sqrt 2)) / 2.  (src/models/gpt2.rs:47-52)"""
    erf = np.vectorize(math.erf, otypes=[F64])
    return x * (1.0 + erf(x / math.sqrt(2.0))) / 2.0


def activation(cfg):
    """gelu_new or gelu, by name only.  (src/models/gpt2.rs:78-97)"""
    name = cfg["activation_function"]
    if name == "gelu_new":
        return gelu_new
    if name == "gelu":
        return gelu_erf
    raise ValueError(name)


def feed_forward(x, w, prefix, act, quant=None):
    """down(act(up(x))).  (src/feed_forward.rs:111-114)"""
    u = act(conv1d(x, w[prefix + "c_fc.weight"], w[prefix + "c_fc.bias"]))
    if quant:
        u = quant(u)
    return conv1d(u, w[prefix + "c_proj.weight"], w[prefix + "c_proj.bias"])


def block(x, cfg, w, layer, key_valid=None, quant=None, taps=None):
    """x + attn(ln_1(x)); then y + mlp(ln_2(y)).  (src/models/gpt2/model.rs:218-270)"""
    p = f"h.{layer}."
    d, nh = cfg["n_embd"], cfg["n_head"]
    eps = cfg["layer_norm_epsilon"]
    n1 = layer_norm(x, w[p + "ln_1.weight"], w[p + "ln_1.bias"], eps)
    if quant:
        n1 = quant(n1)
    qkv = conv1d(n1, w[p + "attn.c_attn.weight"], w[p + "attn.c_attn.bias"])
    if quant:
        qkv = quant(qkv)
    # fused output, three column blocks q | k | v  (src/models/gpt2/checkpoint.rs:131-152)
    q, k, v = (split_heads(qkv[:, i * d:(i + 1) * d], nh) for i in range(3))
    ctx = attention(q, k, v, score_scale(cfg, layer), cfg.get("causal", True), key_valid)
    ctx = merge_heads(ctx)
    if quant:
        ctx = quant(ctx)
    y = x + conv1d(ctx, w[p + "attn.c_proj.weight"], w[p + "attn.c_proj.bias"])
    n2 = layer_norm(y, w[p + "ln_2.weight"], w[p + "ln_2.bias"], eps)
    if quant:
        n2 = quant(n2)
    m = feed_forward(n2, w, p + "mlp.", activation(cfg), quant)
    if taps is not None:
        taps.setdefault("mlp", []).append(m)
    return y + m


def hidden_states(cfg, w, ids, key_valid=None, quant=None, taps=None):
    """Embedding, every block, final norm.  Positions are the physical columns
    0..S-1, padding included.  (src/models/gpt2/model.rs:385-420, src/models/shared/input.rs:345-376)"""
    ids = np.asarray(ids)
    if not (1 <= ids.shape[0] <= cfg["n_positions"]):
        raise ValueError("sequence length outside 1..=n_positions")  # model.rs:431-437
    if ids.min() < 0 or ids.max() >= cfg["vocab_size"]:
        raise ValueError("token id outside the vocabulary")  # shared/input.rs:186-196
    x = embed(ids, np.arange(ids.shape[0]), w["wte.weight"], w["wpe.weight"])
    if taps is not None:
        taps["embedding"] = x
    for layer in range(cfg["n_layer"]):
        x = block(x, cfg, w, layer, key_valid, quant, taps)
        if taps is not None:
            taps.setdefault("residual", []).append(x)
    f = layer_norm(x, w["ln_f.weight"], w["ln_f.bias"], cfg["layer_norm_epsilon"])
    if taps is not None:
        taps["final_norm"] = f
    return f


def logits(cfg, w, ids, key_valid=None, quant=None, taps=None):
    """LN_f(z) @ wte^T at every position of one sequence: [S, V].
    (src/models/gpt2/model.rs:496-513, 550-569)"""
    f = hidden_states(cfg, w, ids, key_valid, quant, taps)
    if quant:
        f = quant(f)
    return f @ w["wte.weight"].T


# --------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------

MASK64 = (1 << 64) - 1


def splitmix64(seed: int, index: int) -> int:
    """Counter-based draw.  (src/generation/random.rs:237-242)"""
    v = (seed + 0x9E3779B97F4A7C15 * ((index + 1) & MASK64)) & MASK64
    v = ((v ^ (v >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    v = ((v ^ (v >> 27)) * 0x94D049BB133111EB) & MASK64
    return v ^ (v >> 31)


def interior_unit(bits: int) -> float:
    """Midpoint of one of 2^23 intervals, strictly inside (0, 1).  (src/generation/random.rs:249-252)"""
    return float(np.float32(((bits >> 41) + 0.5) / float(1 << 23)))


def top_k_filter(z, k):
    """Keep z >= k-th greatest, ties survive.  (src/generation.rs:1199-1209)"""
    boundary = np.sort(z)[::-1][k - 1]
    return np.where(z < boundary, -np.inf, z)


def top_p_filter(z, p):
    """Keep the sorted prefix whose mass before each item is below p.  (src/generation.rs:1224-1234)
    Items tied in value with the last kept item are all kept (the reference leaves
    their order to the sort)."""
    order = np.argsort(-z, kind="stable")
    zs = z[order]
    e = np.exp(zs - zs[0])
    prob = e / e.sum()
    before = np.cumsum(prob) - prob
    keep_sorted = before < p
    boundary = zs[keep_sorted][-1]
    return np.where(z < boundary, -np.inf, z)


def min_p_filter(z, min_p):
    """Keep z >= max + ln(min_p).  (src/generation.rs:1243-1255)"""
    if min_p <= 0:
        return z
    return np.where(z < z.max() + math.log(min_p), -np.inf, z)


def process(z, *, sample, temperature=1.0, top_k=None, top_p=None, min_p=None):
    """temperature, then top-k, top-p, min-p; only when sampling.  (src/generation.rs:605-652)"""
    z = np.asarray(z, dtype=F64)
    if not sample:
        return z
    z = z / temperature
    if top_k is not None:
        z = top_k_filter(z, top_k)
    if top_p is not None:
        z = top_p_filter(z, top_p)
    if min_p is not None:
        z = min_p_filter(z, min_p)
    return z


def log_softmax(z):
    m = z.max()
    return z - m - math.log(np.exp(z - m).sum())


def select(z, *, sample, u=None):
    """argmax, or #{k : c_k < u * c_(V-1)} on the running sums of softmax(z).
    (src/generation.rs:655-664, 1126-1165)  Returns (id, log-probability)."""
    if not sample:
        tok = int(np.argmax(z))
    else:
        e = np.exp(z - z.max())
        c = np.cumsum(e / e.sum())
        tok = int((c < u * c[-1]).sum())
    return tok, float(log_softmax(z)[tok])


def generate(cfg, w, prompt, max_new_tokens, *, sample=False, temperature=1.0, seed=0,
             stream=0, eos=(), top_k=None, top_p=None, min_p=None, quant=None):
    """Recomputes the whole sequence for every new token.  The uniform of draw k of
    this sequence is splitmix64(stream seed, k); `stream` is the seed of the
    sequence's own stream as the engine derives it."""
    ids = list(prompt)
    out, logp = [], []
    for k in range(max_new_tokens):
        z = logits(cfg, w, ids, quant=quant)[-1]
        z = process(z, sample=sample, temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p)
        u = interior_unit(splitmix64(stream, k)) if sample else None
        tok, lp = select(z, sample=sample, u=u)
        out.append(tok)
        logp.append(lp)
        ids.append(tok)
        if tok in eos:
            break
    return out, logp
