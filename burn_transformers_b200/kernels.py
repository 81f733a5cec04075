"""Python face of the CUDA kernel library: loads it, checks arguments, launches on torch's stream.

There is no fallback: if the library cannot be built or loaded, or a tensor lies on the host,
the call raises.  Tensors are passed as raw device pointers; shapes and dtypes are checked here
so that a kernel never sees a size it was not written for.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .errors import KernelError, ShapeError

_LIB = None
DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
ACTIVATIONS = {None: 0, "none": 0, "gelu_new": 1, "gelu_tanh": 1, "gelu": 2, "gelu_erf": 2}
PAGE_SIZE = 64


def library() -> ctypes.CDLL:
    """The loaded kernel library; builds it on first use."""
    global _LIB
    if _LIB is None:
        from .csrc.build import build
        path = build()
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as error:
            raise KernelError(f"cannot load the CUDA kernel library {path}: {error}") from None
        lib.bt_last_error.restype = ctypes.c_char_p
        lib.bt_attention_decode_scratch_floats.restype = c_longlong
        lib.bt_launch_count.restype = c_longlong
        if lib.bt_abi_version() != 1:
            raise KernelError(f"{path} has an unexpected interface version")
        _LIB = lib
    return _LIB if _PROFILE is None else _Bracketed(_LIB, _PROFILE)


class KernelProfile:
    """Times every launch of the library on the device while it is active (`with KernelProfile() as p: ...`).

    Each launch is bracketed by two CUDA events on the launching stream; `summary()` waits for them and returns, per
    kernel, the number of launches, the time, and what the wrappers said the launches had to do (floating-point
    operations and bytes that must move), from which achieved TFLOP/s and GB/s follow.  Launches recorded into a
    CUDA graph cannot be timed this way: profile steps that run their kernels directly."""

    SKIP = ("bt_last_error", "bt_launch_count", "bt_abi_version", "bt_tensor_map", "bt_decode_flow_plan",
            "bt_decode_flow_phase_bytes", "bt_attention_decode_scratch_floats")

    def __init__(self):
        self.records = []          # (name, start event, stop event, flops, bytes)
        self.pending = (0.0, 0.0)

    def __enter__(self):
        global _PROFILE
        _PROFILE = self
        return self

    def __exit__(self, *exc):
        global _PROFILE
        _PROFILE = None

    def summary(self) -> list[dict]:
        torch.cuda.synchronize()
        rows: dict[str, dict] = {}
        for name, start, stop, flops, nbytes in self.records:
            row = rows.setdefault(name, {"kernel": name, "launches": 0, "ms": 0.0, "flops": 0.0, "bytes": 0.0})
            row["launches"] += 1
            row["ms"] += start.elapsed_time(stop)
            row["flops"] += flops
            row["bytes"] += nbytes
        total = sum(r["ms"] for r in rows.values()) or 1.0
        out = []
        for row in sorted(rows.values(), key=lambda r: -r["ms"]):
            seconds = row["ms"] * 1e-3
            row["share"] = row["ms"] / total
            row["tflops"] = row["flops"] / seconds / 1e12 if seconds > 0 and row["flops"] else None
            row["gbs"] = row["bytes"] / seconds / 1e9 if seconds > 0 and row["bytes"] else None
            out.append(row)
        return out


class _Bracketed:
    """The library as the wrappers see it while a profile is active: every launch between two events and inside
    an NVTX range of the kernel's name."""

    def __init__(self, lib, profile):
        self._lib, self._profile = lib, profile

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        if name.endswith("_supports") or name.startswith(KernelProfile.SKIP):
            return fn
        profile = self._profile

        def launch(*args):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.nvtx.range_push(name)      # (a timeline tool shows the same brackets by name)
            start.record()
            code = fn(*args)
            stop.record()
            torch.cuda.nvtx.range_pop()
            flops, nbytes = profile.pending
            profile.pending = (0.0, 0.0)
            profile.records.append((name[3:] if name.startswith("bt_") else name, start, stop, flops, nbytes))
            return code
        return launch


_PROFILE: KernelProfile | None = None


def _work(flops: float = 0.0, nbytes: float = 0.0) -> None:
    """What the next launch has to do (for a profile; costs nothing otherwise)."""
    if _PROFILE is not None:
        _PROFILE.pending = (float(flops), float(nbytes))


def _linear_work(m, n, k, a, w, out) -> None:
    if _PROFILE is not None:
        _work(2.0 * m * n * k, m * k * (a.element_size() if hasattr(a, "element_size") else 4) + n * k * w.element_size()
              + m * n * out.element_size())


def launch_count() -> int:
    """Kernel launches issued through the library so far (a launch recorded into a CUDA graph counts once)."""
    return int(library().bt_launch_count())


def _check(code: int) -> None:
    if code != 0:
        raise KernelError(library().bt_last_error().decode(errors="replace"))


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    """Device, layout, element type and extents of one argument (None in `shape` leaves an extent free)."""
    try:
        ok = t.is_cuda and t.is_contiguous()
    except AttributeError:
        raise ShapeError(f"{name}: expected a tensor, found {type(t).__name__}") from None
    if not ok:
        if not t.is_cuda:
            raise KernelError(f"{name}: lies on {t.device}; the kernels of this library run on a CUDA device only")
        raise ShapeError(f"{name}: must be contiguous")
    if dtype is not None and t.dtype is not dtype:
        if not isinstance(dtype, (tuple, list)) or t.dtype not in dtype:
            raise ShapeError(f"{name}: expected dtype {dtype}, found {t.dtype}")
    if shape is not None:
        got = t.shape
        if len(shape) != len(got):
            raise ShapeError(f"{name}: expected shape {list(shape)}, found {list(got)}")
        for want, have in zip(shape, got):
            if want is not None and want != have:
                raise ShapeError(f"{name}: expected shape {list(shape)}, found {list(got)}")


def _code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dtype]
    except KeyError:
        raise ShapeError(f"unsupported element type {dtype}") from None


# --------------------------------------------------------------------------------------------

def embed(tokens, positions, wte, wpe, out, status=None):
    """out[t] = wte[tokens[t]] (+ wpe[positions[t]]) into the 32-bit residual stream."""
    n = tokens.shape[0]
    vocab, width = wte.shape
    _need(tokens, "tokens", torch.int32, (n,))
    _need(wte, "wte", (torch.float32, torch.bfloat16))
    _need(out, "out", torch.float32, (None, width))
    n_pos = 0
    if wpe is not None:
        _need(positions, "positions", torch.int32, (n,))
        _need(wpe, "wpe", wte.dtype, (None, width))
        n_pos = wpe.shape[0]
    if out.shape[0] < n:
        raise ShapeError(f"out: {out.shape[0]} rows for {n} tokens")
    _work(0.0, n * width * (wte.element_size() * (2 if wpe is not None else 1) + 4))
    _check(library().bt_embed(_ptr(tokens), _ptr(positions if wpe is not None else None), _ptr(wte), _ptr(wpe), _ptr(out),
                              c_int(n), c_int(width), c_int(vocab), c_int(n_pos), c_int(_code(wte.dtype)),
                              _ptr(status), _stream()))


def layernorm(x, gamma, beta, out, eps: float, rows=None, n_rows=None):
    """out[r] = LayerNorm(x[rows[r]] or x[r]); x is 32-bit, out is 32-bit or bfloat16."""
    width = x.shape[-1]
    _need(x, "x", torch.float32, (None, width))
    _need(gamma, "gamma", torch.float32, (width,))
    if beta is not None:
        _need(beta, "beta", torch.float32, (width,))
    n = n_rows if n_rows is not None else (rows.shape[0] if rows is not None else x.shape[0])
    if rows is not None:
        _need(rows, "rows", torch.int32)
    _need(out, "out", (torch.float32, torch.bfloat16), (None, width))
    if out.shape[0] < n:
        raise ShapeError(f"out: {out.shape[0]} rows for {n} rows")
    _work(0.0, n * width * (4 + out.element_size()))
    _check(library().bt_layernorm(_ptr(x), _ptr(rows), _ptr(gamma), _ptr(beta), _ptr(out), c_int(n), c_int(width),
                                  c_float(eps), c_int(_code(out.dtype)), _stream()))


def linear_simt(a, w, bias, out, *, m=None, w_is_nk=False, activation=None, residual=None):
    """out = act(a @ w + bias) (+ residual) with 32-bit fused multiply-adds.

    a: [M, K]; w: [K, N] (or [N, K] when w_is_nk); bias: [N] float32 or None; residual: [M, N]
    float32 (may be `out` itself); out: [M, N] float32 or a's dtype.
    """
    k = a.shape[1]
    n = w.shape[0] if w_is_nk else w.shape[1]
    m = a.shape[0] if m is None else m
    _need(a, "a", (torch.float32, torch.bfloat16), (None, k))
    _need(w, "w", a.dtype, (n, k) if w_is_nk else (k, n))
    _need(out, "out", (torch.float32, a.dtype), (None, n))
    if bias is not None:
        _need(bias, "bias", torch.float32, (n,))
    if residual is not None:
        _need(residual, "residual", torch.float32, (None, n))
    if a.shape[0] < m or out.shape[0] < m:
        raise ShapeError(f"linear: {m} rows asked of a[{a.shape[0]}] and out[{out.shape[0]}]")
    if activation not in ACTIVATIONS:
        raise ShapeError(f"linear: unknown activation {activation!r}")
    _linear_work(m, n, k, a, w, out)
    _check(library().bt_linear_simt(_ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), c_int(m), c_int(n), c_int(k),
                                    c_int(1 if w_is_nk else 0), c_int(ACTIVATIONS[activation]), c_int(_code(a.dtype)),
                                    c_int(_code(out.dtype)), _stream()))


def linear_skinny_supports(m, n, k, w_is_nk, fuse_ln) -> bool:
    return _supports("bt_linear_skinny_supports", m, n, k, 1 if w_is_nk else 0, 1 if fuse_ln else 0)


def linear_skinny(a, w, bias, out, *, m, w_is_nk=False, activation=None, residual=None, norm=None, split=0):
    """out[:m] = act(rows @ w + bias) (+ residual) for at most 64 bfloat16 rows.

    rows are `a` (bfloat16 [M, K]) or, when `norm` = (x32, gamma, beta, eps, row_index) is given and `a` is None,
    LayerNorm(x32[row_index]) formed inside the kernel."""
    n = w.shape[0] if w_is_nk else w.shape[1]
    k = w.shape[1] if w_is_nk else w.shape[0]
    _need(w, "w", torch.bfloat16, (n, k) if w_is_nk else (k, n))
    _need(out, "out", (torch.float32, torch.bfloat16), (None, n))
    if out.shape[0] < m:
        raise ShapeError(f"linear_skinny: {m} rows asked of out[{out.shape[0]}]")
    if bias is not None:
        _need(bias, "bias", torch.float32, (n,))
    if residual is not None:
        _need(residual, "residual", torch.float32, (None, n))
    if activation not in ACTIVATIONS:
        raise ShapeError(f"linear_skinny: unknown activation {activation!r}")
    x32 = gamma = beta = rows = None
    eps = 0.0
    if norm is not None:
        x32, gamma, beta, eps, rows = norm
        _need(x32, "x32", torch.float32, (None, k))
        _need(gamma, "gamma", torch.float32, (k,))
        if beta is not None:
            _need(beta, "beta", torch.float32, (k,))
        if rows is not None:
            _need(rows, "rows", torch.int32)
        elif x32.shape[0] < m:
            raise ShapeError(f"linear_skinny: {m} rows asked of x32[{x32.shape[0]}]")
    else:
        _need(a, "a", torch.bfloat16, (None, k))
        if a.shape[0] < m:
            raise ShapeError(f"linear_skinny: {m} rows asked of a[{a.shape[0]}]")
    _linear_work(m, n, k, w, w, out)
    _check(library().bt_linear_skinny(_ptr(a if norm is None else None), _ptr(x32), _ptr(rows), _ptr(gamma), _ptr(beta),
                                      c_float(eps), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), c_int(m), c_int(n),
                                      c_int(k), c_int(1 if w_is_nk else 0), c_int(ACTIVATIONS[activation]),
                                      c_int(1 if out.dtype == torch.float32 else 0), c_int(split), _stream()))


def linear_mid(a, w, bias, out, *, m, activation=None, residual=None, split=0):
    """out[:m] = act(a[:m] @ w^T + bias) (+ residual) for at most 64 bfloat16 rows and weights stored [N, K]: the
    product made for 17 to 64 rows (a block per 16 columns over the whole of K, operands through a ring of
    tensor-map copies)."""
    n, k = w.shape
    _need(w, "w", torch.bfloat16, (n, k))
    _need(a, "a", torch.bfloat16, (None, k))
    _need(out, "out", (torch.float32, torch.bfloat16), (None, n))
    if a.shape[0] < m or out.shape[0] < m:
        raise ShapeError(f"linear_mid: {m} rows asked of a[{a.shape[0]}], out[{out.shape[0]}]")
    if bias is not None:
        _need(bias, "bias", torch.float32, (n,))
    if residual is not None:
        _need(residual, "residual", torch.float32, (None, n))
    if activation not in ACTIVATIONS:
        raise ShapeError(f"linear_mid: unknown activation {activation!r}")
    _linear_work(m, n, k, a, w, out)
    _check(library().bt_linear_mid(_ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), _ptr(kernel_status(a.device)),
                                   c_int(m), c_int(n), c_int(k), c_int(ACTIVATIONS[activation]),
                                   c_int(1 if out.dtype == torch.float32 else 0), c_int(split), _stream()))


def linear_mid_supports(m, n, k) -> bool:
    return _supports("bt_linear_mid_supports", m, n, k)


_SUPPORTS: dict = {}


def _supports(name: str, *args) -> bool:
    """Answers of the library's pure `..._supports` questions, remembered."""
    key = (name, args)
    hit = _SUPPORTS.get(key)
    if hit is None:
        hit = bool(getattr(library(), name)(*[c_int(int(a)) for a in args]))
        _SUPPORTS[key] = hit
    return hit


def linear_tcgen05_supports(m, n, k) -> bool:
    return _supports("bt_linear_tcgen05_supports", m, n, k)


def linear_tcgen05(a, w, bias, out, *, m, activation=None, residual=None):
    """out[:m] = act(a[:m] @ w^T + bias) (+ residual) on the tcgen05 tensor cores; a [M, K] and w [N, K] bfloat16."""
    n, k = w.shape
    _need(a, "a", torch.bfloat16, (None, k))
    _need(w, "w", torch.bfloat16, (n, k))
    _need(out, "out", (torch.float32, torch.bfloat16), (None, n))
    if a.shape[0] < m or out.shape[0] < m:
        raise ShapeError(f"linear_tcgen05: {m} rows asked of a[{a.shape[0]}] and out[{out.shape[0]}]")
    if bias is not None:
        _need(bias, "bias", torch.float32, (n,))
    if residual is not None:
        _need(residual, "residual", torch.float32, (None, n))
    if activation not in ACTIVATIONS:
        raise ShapeError(f"linear_tcgen05: unknown activation {activation!r}")
    _linear_work(m, n, k, a, w, out)
    _check(library().bt_linear_tcgen05(_ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out),
                                       _ptr(kernel_status(a.device)), c_int(m), c_int(n), c_int(k),
                                       c_int(ACTIVATIONS[activation]), c_int(1 if out.dtype == torch.float32 else 0),
                                       _stream()))


def linear_few_tcgen05_supports(m, n, k) -> bool:
    return _supports("bt_linear_few_tcgen05_supports", m, n, k)


def linear_few_tcgen05(a, w, bias, out, *, m, activation=None, residual=None, split=0):
    """out[:m] = act(a[:m] @ w^T + bias) (+ residual) for at most 128 bfloat16 rows and weights stored [N, K], on the
    tcgen05 tensor cores with the weights on their M side: the product for few rows over large weights (a block per
    128 columns and slice of K, the slices of a cluster summed through distributed shared memory)."""
    n, k = w.shape
    _need(a, "a", torch.bfloat16, (None, k))
    _need(w, "w", torch.bfloat16, (n, k))
    _need(out, "out", (torch.float32, torch.bfloat16), (None, n))
    if a.shape[0] < m or out.shape[0] < m:
        raise ShapeError(f"linear_few_tcgen05: {m} rows asked of a[{a.shape[0]}] and out[{out.shape[0]}]")
    if bias is not None:
        _need(bias, "bias", torch.float32, (n,))
    if residual is not None:
        _need(residual, "residual", torch.float32, (None, n))
    if activation not in ACTIVATIONS:
        raise ShapeError(f"linear_few_tcgen05: unknown activation {activation!r}")
    _linear_work(m, n, k, a, w, out)
    _check(library().bt_linear_few_tcgen05(_ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out),
                                           _ptr(kernel_status(a.device)), c_int(m), c_int(n), c_int(k),
                                           c_int(ACTIVATIONS[activation]), c_int(1 if out.dtype == torch.float32 else 0),
                                           c_int(split), _stream()))


def linear_stream_supports(m, n, k, fuse_ln) -> bool:
    return _supports("bt_linear_stream_supports", m, n, k, 1 if fuse_ln else 0)


def linear_stream(a, w, bias, out, *, m, activation=None, residual=None, norm=None, warps_k=0):
    """out[:m] = act(rows @ w^T + bias) (+ residual) for at most 64 bfloat16 rows; w is [N, K].

    rows are `a` (bfloat16 [M, K]) or, when `norm` = (x32, gamma, beta, eps, row_index) is given and `a` is None,
    LayerNorm(x32[row_index]) formed inside the kernel (at most 16 rows)."""
    n, k = w.shape
    _need(w, "w", torch.bfloat16, (n, k))
    _need(out, "out", (torch.float32, torch.bfloat16), (None, n))
    if out.shape[0] < m:
        raise ShapeError(f"linear_stream: {m} rows asked of out[{out.shape[0]}]")
    if bias is not None:
        _need(bias, "bias", torch.float32, (n,))
    if residual is not None:
        _need(residual, "residual", torch.float32, (None, n))
    if activation not in ACTIVATIONS:
        raise ShapeError(f"linear_stream: unknown activation {activation!r}")
    x32 = gamma = beta = rows = None
    eps = 0.0
    if norm is not None:
        x32, gamma, beta, eps, rows = norm
        _need(x32, "x32", torch.float32, (None, k))
        _need(gamma, "gamma", torch.float32, (k,))
        if beta is not None:
            _need(beta, "beta", torch.float32, (k,))
        if rows is not None:
            _need(rows, "rows", torch.int32)
        elif x32.shape[0] < m:
            raise ShapeError(f"linear_stream: {m} rows asked of x32[{x32.shape[0]}]")
    else:
        _need(a, "a", torch.bfloat16, (None, k))
        if a.shape[0] < m:
            raise ShapeError(f"linear_stream: {m} rows asked of a[{a.shape[0]}]")
    _linear_work(m, n, k, w, w, out)
    _check(library().bt_linear_stream(_ptr(a if norm is None else None), _ptr(x32), _ptr(rows), _ptr(gamma), _ptr(beta),
                                      c_float(eps), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), c_int(m), c_int(n),
                                      c_int(k), c_int(ACTIVATIONS[activation]),
                                      c_int(1 if out.dtype == torch.float32 else 0), c_int(warps_k), _stream()))


def kv_append(proj, k_offset, v_offset, positions, token_seq, ctx_len, table, table_len, k_pool, v_pool,
              n_tokens, n_kv_heads, head_dim):
    """Copies the new tokens' key and value channels of `proj` rows into the layer's pages."""
    _need(proj, "proj", (torch.float32, torch.bfloat16))
    _need(k_pool, "k_pool", proj.dtype)
    _need(v_pool, "v_pool", proj.dtype)
    _need(table, "table", torch.int32)
    _work(0.0, 4.0 * n_tokens * n_kv_heads * head_dim * proj.element_size())
    _check(library().bt_kv_append(_ptr(proj), c_longlong(proj.shape[1]), c_int(k_offset), c_int(v_offset),
                                  _ptr(positions), _ptr(token_seq), _ptr(ctx_len), _ptr(table), c_int(table.shape[1]),
                                  c_int(table_len), c_int(PAGE_SIZE), _ptr(k_pool), _ptr(v_pool), c_int(n_tokens),
                                  c_int(n_kv_heads), c_int(head_dim), c_int(_code(proj.dtype)), _stream()))


def attention_prefill_simt(q_proj, out, seq_start, past_len, n_seqs, max_new, n_heads, n_kv_heads, head_dim, scale,
                           *, causal=True, window=0, k_pool=None, v_pool=None, table=None, table_len=0,
                           k_offset=None, v_offset=None):
    """Attention of several new tokens per sequence.

    Queries are the first n_heads*head_dim channels of `q_proj` rows.  Keys and values come either
    from the pages (`k_pool`, `v_pool`, `table`) or, when `table` is None, from the channels
    `k_offset`, `v_offset` of the same rows (sequences that start at position 0).
    """
    _need(q_proj, "q_proj", (torch.float32, torch.bfloat16))
    _need(out, "out", q_proj.dtype, (None, n_heads * head_dim))
    stride = q_proj.shape[1]
    es = q_proj.element_size()
    if table is None:
        k_ptr = c_void_p(q_proj.data_ptr() + k_offset * es)
        v_ptr = c_void_p(q_proj.data_ptr() + v_offset * es)
        t_ptr, t_stride = c_void_p(0), 0
    else:
        _need(k_pool, "k_pool", q_proj.dtype)
        _need(v_pool, "v_pool", q_proj.dtype)
        _need(table, "table", torch.int32)
        k_ptr, v_ptr, t_ptr, t_stride = _ptr(k_pool), _ptr(v_pool), _ptr(table), table.shape[1]
    _check(library().bt_attention_prefill_simt(
        _ptr(q_proj), c_longlong(stride), k_ptr, v_ptr, t_ptr, c_int(t_stride), c_int(table_len), c_int(PAGE_SIZE),
        c_longlong(stride), _ptr(out), _ptr(seq_start), _ptr(past_len), c_int(n_seqs), c_int(max_new), c_int(n_heads),
        c_int(n_kv_heads), c_int(head_dim), c_float(scale), c_int(1 if causal else 0), c_int(window),
        c_int(_code(q_proj.dtype)), _stream()))


def attention_prefill(q_proj, out, seq_start, past_len, n_seqs, max_new, n_heads, n_kv_heads, head_dim, scale, *,
                      impl=None, **kw):
    """Attention of several new tokens per sequence.  bfloat16 with a head size the kernels are built for runs on
    tensor cores (tcgen05 with the scores in tensor memory), everything else with the plain 32-bit kernel.
    `impl` ("tcgen05", "simt") asks for one kernel by name.  Arguments as attention_prefill_simt."""
    bf16 = q_proj.dtype == torch.bfloat16
    if impl is None:
        if bf16 and _supports("bt_attention_prefill_tcgen05_supports", head_dim, PAGE_SIZE):
            impl = "tcgen05"
        else:
            impl = "simt"
    if impl == "tcgen05":
        return _attention_prefill_tcgen05(q_proj, out, seq_start, past_len, n_seqs, max_new, n_heads, n_kv_heads,
                                          head_dim, scale, **kw)
    return attention_prefill_simt(q_proj, out, seq_start, past_len, n_seqs, max_new, n_heads, n_kv_heads, head_dim,
                                  scale, **kw)


def _attention_prefill_tcgen05(q_proj, out, seq_start, past_len, n_seqs, max_new, n_heads, n_kv_heads, head_dim, scale,
                               *, causal=True, window=0, k_pool=None, v_pool=None, table=None, table_len=0,
                               k_offset=None, v_offset=None):
    _need(q_proj, "q_proj", torch.bfloat16)
    _need(out, "out", torch.bfloat16, (None, n_heads * head_dim))
    stride = q_proj.shape[1]
    if table is None:
        k_ptr = c_void_p(q_proj.data_ptr() + k_offset * 2)
        v_ptr = c_void_p(q_proj.data_ptr() + v_offset * 2)
        t_ptr, t_stride, pages = c_void_p(0), 0, 0
    else:
        _need(k_pool, "k_pool", torch.bfloat16)
        _need(v_pool, "v_pool", torch.bfloat16)
        _need(table, "table", torch.int32)
        k_ptr, v_ptr, t_ptr, t_stride, pages = _ptr(k_pool), _ptr(v_pool), _ptr(table), table.shape[1], k_pool.shape[0]
    _check(library().bt_attention_prefill_tcgen05(
        _ptr(q_proj), c_longlong(q_proj.shape[0]), c_longlong(stride), k_ptr, v_ptr, c_longlong(pages), t_ptr,
        c_int(t_stride), c_int(table_len), c_int(PAGE_SIZE), _ptr(out), _ptr(kernel_status(q_proj.device)),
        _ptr(seq_start), _ptr(past_len), c_int(n_seqs), c_int(max_new), c_int(n_heads), c_int(n_kv_heads),
        c_int(head_dim), c_float(scale), c_int(1 if causal else 0), c_int(window), _stream()))


def attention_decode_supports(head_dim: int, row_stride: int, dtype) -> bool:
    """Whether the decode-attention kernels take this head size: they move rows as 16-byte pieces, so a head and a
    projection row must be whole pieces (8 bfloat16 or, as the kernel is built, 8 floats), at most 256 wide."""
    return head_dim % 8 == 0 and row_stride % 8 == 0 and 0 < head_dim <= 256


def attention_decode_scratch_floats(n_seqs, n_heads, head_dim, n_splits) -> int:
    return int(library().bt_attention_decode_scratch_floats(c_int(n_seqs), c_int(n_heads), c_int(head_dim), c_int(n_splits)))


_TICKETS: dict = {}


def _tickets(device, count: int) -> torch.Tensor:
    """Zeroed counters for the decode attention's merge; the kernel leaves them zero, so they are made once."""
    t = _TICKETS.get(device)
    if t is None or t.numel() < count:
        t = torch.zeros(max(count, 1 << 14), dtype=torch.int32, device=device)
        _TICKETS[device] = t
    return t


_STATUS: dict = {}


def kernel_status(device) -> torch.Tensor:
    """One int per device that a kernel sets when a bounded wait of its own ran out (see attention_decode)."""
    t = _STATUS.get(device)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _STATUS[device] = t
    return t


_STATUS_TEXT = {1: "decode attention gave up waiting for a copy of cache pages",
                2: "the tcgen05 matrix product gave up waiting for a stage of its pipeline",
                3: "the fused decode step gave up at a grid barrier or waiting for cache pages",
                4: "the fused decode step met a token id or position outside its table",
                5: "the matrix product for 17 to 64 rows gave up waiting for a stage of its pipeline",
                6: "the tcgen05 prefill attention gave up waiting for a stage of its pipeline (or found its shared memory "
                   "misaligned)",
                7: "the tcgen05 matrix product for few rows gave up waiting for a stage of its pipeline"}


def check_status(device) -> None:
    """Raises if a kernel on `device` reported that one of its bounded waits ran out (its results are then not to be
    trusted), and clears the report.  Reads one int from the device: call it where the host waits anyway."""
    t = _STATUS.get(device)
    if t is None:
        return
    code = int(t.item())
    if code:
        t.zero_()
        raise KernelError(_STATUS_TEXT.get(code, f"a kernel reported status {code}"))


def attention_decode(q_proj, out, k_pool, v_pool, table, table_len, ctx_len, n_seqs, n_heads, n_kv_heads, head_dim,
                     scale, *, max_ctx, window=0, n_splits=1, scratch=None, new_kv_offsets=None, merge_in_scratch=False,
                     tensor_cores=True):
    """Attention of one new token per sequence over that sequence's pages.

    bfloat16 with a head size of 16..128 in steps of 16 runs on tensor cores (`tensor_cores=False` keeps it on
    the 32-bit multiply-add kernel that every other case takes).

    `max_ctx`: no sequence of the call is longer than this.  `new_kv_offsets` = (k_offset, v_offset): the new
    token's key and value are channels of the same `q_proj` rows; the kernel reads them from there and files
    them in the pages itself.  None: the pages already hold them.  Up to 8 splits merge inside a thread-block
    cluster; more (or `merge_in_scratch`) need `scratch`."""
    _need(q_proj, "q_proj", (torch.float32, torch.bfloat16))
    _need(out, "out", q_proj.dtype, (None, n_heads * head_dim))
    _need(k_pool, "k_pool", q_proj.dtype)
    _need(v_pool, "v_pool", q_proj.dtype)
    _need(table, "table", torch.int32)
    tickets = None
    use_mma = (tensor_cores and q_proj.dtype == torch.bfloat16
               and bool(library().bt_attention_decode_mma_supports(c_int(head_dim))))
    if n_splits > 1 and (n_splits > 8 or merge_in_scratch):
        need = attention_decode_scratch_floats(n_seqs, n_heads, head_dim, n_splits)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise ShapeError(f"attention_decode: {n_splits} splits need {need} floats of scratch")
        tickets = _tickets(q_proj.device, n_seqs * n_heads)
    es = q_proj.element_size()
    new_k = new_v = c_void_p(0)
    if new_kv_offsets is not None:
        new_k = c_void_p(q_proj.data_ptr() + new_kv_offsets[0] * es)
        new_v = c_void_p(q_proj.data_ptr() + new_kv_offsets[1] * es)
    if use_mma:
        _check(library().bt_attention_decode_mma(
            _ptr(q_proj), c_longlong(q_proj.shape[1]), new_k, new_v, _ptr(k_pool), _ptr(v_pool),
            c_longlong(k_pool.numel() // (n_kv_heads * PAGE_SIZE * head_dim)), _ptr(table), c_int(table.shape[1]),
            c_int(table_len), _ptr(out), _ptr(scratch), _ptr(tickets), _ptr(kernel_status(q_proj.device)), _ptr(ctx_len),
            c_int(n_seqs), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_float(scale), c_int(window),
            c_int(n_splits), c_int(max_ctx), c_int(1 if merge_in_scratch else 0), _stream()))
        return
    _check(library().bt_attention_decode(
        _ptr(q_proj), c_longlong(q_proj.shape[1]), new_k, new_v, _ptr(k_pool), _ptr(v_pool), _ptr(table),
        c_int(table.shape[1]), c_int(table_len), c_int(PAGE_SIZE), _ptr(out), _ptr(scratch), _ptr(tickets),
        _ptr(kernel_status(q_proj.device)), _ptr(ctx_len), c_int(n_seqs), c_int(n_heads), c_int(n_kv_heads),
        c_int(head_dim), c_float(scale), c_int(window), c_int(n_splits), c_int(max_ctx),
        c_int(1 if merge_in_scratch else 0), c_int(_code(q_proj.dtype)), _stream()))


def sample(logits, n_rows, *, do_sample, temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, uniforms=None,
           stream_seeds=None, counters=None, out_ids=None, out_logp=None):
    """Selects one token per row of 32-bit logits; writes ids (int32) and log-probabilities (float32).

    Sampling takes one uniform per row from `uniforms`, or draws it on the device as draw `counters[r]` of the
    SplitMix64 stream `stream_seeds[r]` (int64 tensor holding the unsigned seeds' bits)."""
    _need(logits, "logits", torch.float32)
    vocab = logits.shape[1]
    _need(out_ids, "out_ids", torch.int32)
    _need(out_logp, "out_logp", torch.float32)
    if do_sample and stream_seeds is not None:
        _need(stream_seeds, "stream_seeds", torch.int64)
        _need(counters, "counters", torch.int32)
    elif do_sample:
        _need(uniforms, "uniforms", torch.float32)
    _check(library().bt_sample(_ptr(logits), c_longlong(logits.stride(0)), c_int(n_rows), c_int(vocab),
                               c_int(1 if do_sample else 0), c_float(temperature), c_int(top_k or 0),
                               c_float(1.0 if top_p is None else top_p), c_float(0.0 if min_p is None else min_p),
                               _ptr(uniforms), _ptr(stream_seeds), _ptr(counters), _ptr(out_ids), _ptr(out_logp),
                               _stream()))


def advance(ids, tokens, positions, past_len, ctx_len, counters, n):
    """tokens <- ids; positions, past_len, ctx_len and counters += 1 (all int32 device tensors of n entries)."""
    for name, t in (("ids", ids), ("tokens", tokens), ("positions", positions), ("past_len", past_len),
                    ("ctx_len", ctx_len), ("counters", counters)):
        _need(t, name, torch.int32)
    _check(library().bt_advance(_ptr(ids), _ptr(tokens), _ptr(positions), _ptr(past_len), _ptr(ctx_len), _ptr(counters),
                                c_int(n), _stream()))


def logit_edits(logits, rows, tokens, vals, n_edits):
    """Applies sparse edits (row, token, [add, repetition, subtract, ban]) to 32-bit logits in place."""
    _need(logits, "logits", torch.float32)
    _check(library().bt_logit_edits(_ptr(logits), c_longlong(logits.stride(0)), _ptr(rows), _ptr(tokens), _ptr(vals),
                                    c_int(n_edits), c_int(logits.shape[1]), _stream()))
