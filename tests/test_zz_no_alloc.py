"""The decode-attention entry point that allocates nothing, called through its exported C symbol.

`bt_attention_decode_static` is for callers that cannot get device memory of their own (a plug-in that is
handed only its inputs and outputs, a serving loop that forbids cudaMalloc after start-up): it keeps the
scratch for its splits in an array inside the library.  It must give what `bt_attention_decode` gives with
caller-owned scratch.  Two calls in a row, with different inputs and split counts, check that nothing left
in the shared array by the first call leaks into the second.  This file is collected last on purpose.
"""
import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

from burn_transformers_b200 import kernels

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = kernels.PAGE_SIZE
STATIC_FLOATS = 1 << 20


def paged(lengths, n_kv_heads, head_dim, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    width = -(-max(lengths) // PAGE)
    n_pages = len(lengths) * width
    order = torch.randperm(n_pages, generator=g)
    table = order.view(len(lengths), width).to(torch.int32)
    k = torch.randn(n_pages, n_kv_heads, PAGE, head_dim, generator=g).to(dtype)
    v = torch.randn(n_pages, n_kv_heads, PAGE, head_dim, generator=g).to(dtype)
    return k.to(DEV), v.to(DEV), table.to(DEV)


def call_static(lib, q, k, v, table, ctx_len, out, n_heads, n_kv_heads, head_dim, scale, window, splits, table_len=None):
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib.bt_attention_decode_static(
        c_void_p(q.data_ptr()), c_longlong(q.shape[1]), c_void_p(k.data_ptr()), c_void_p(v.data_ptr()),
        c_void_p(table.data_ptr()), c_int(table.shape[1]), c_int(table_len or table.shape[1]), c_int(PAGE),
        c_void_p(out.data_ptr()),
        c_void_p(ctx_len.data_ptr()), c_int(q.shape[0]), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim),
        c_float(scale), c_int(window), c_int(splits), c_int(kernels.DTYPE_CODE[q.dtype]), stream)


def plain_attention(q, k, v, table, lengths, hq, hkv, hd, scale, window, table_len=None):
    """The same attention written out with torch in float64: position p of sequence s lies in row p % 64 of page
    table[s][(p // 64) % table_len]."""
    table_len = table_len or table.shape[1]
    out = torch.zeros(len(lengths), hq * hd, dtype=torch.float64)
    k, v, q, table = k.double().cpu(), v.double().cpu(), q.double().cpu(), table.cpu()
    for s, n in enumerate(lengths):
        lo = max(0, n - window) if window else 0
        pos = torch.arange(lo, n)
        pages = table[s][(pos // PAGE) % table_len].long()
        for h in range(hq):
            kh = h // (hq // hkv)
            keys, values = k[pages, kh, pos % PAGE], v[pages, kh, pos % PAGE]
            weights = torch.softmax(keys @ q[s, h * hd:(h + 1) * hd] * scale, 0)
            out[s, h * hd:(h + 1) * hd] = weights @ values
    return out


def device_free_bytes():
    """Free device memory as the driver counts it: an allocation by anybody in the process, torch's allocator or a
    cudaMalloc inside the library, shows here."""
    return torch.cuda.mem_get_info()[0]


@pytest.mark.parametrize("dtype, tol", [(torch.float32, 2e-6), (torch.bfloat16, 4e-3)])
def test_static_scratch_entry_point_matches_the_ordinary_one(dtype, tol):
    lib = kernels.library()
    lib.bt_attention_decode_static.restype = c_int
    lib.bt_attention_decode_static_status.restype = c_int
    calls = [dict(lengths=[700, 65, 1, 300], hq=6, hkv=2, hd=64, window=0, splits=5, seed=1),
             dict(lengths=[129, 500], hq=4, hkv=4, hd=48, window=100, splits=3, seed=2)]
    for c in calls:
        k, v, table = paged(c["lengths"], c["hkv"], c["hd"], dtype, c["seed"])
        n = len(c["lengths"])
        q = torch.randn(n, c["hq"] * c["hd"], generator=torch.Generator().manual_seed(c["seed"])).to(dtype).to(DEV)
        ctx_len = torch.tensor(c["lengths"], dtype=torch.int32, device=DEV)
        want = torch.empty(n, c["hq"] * c["hd"], device=DEV, dtype=dtype)
        scratch = torch.empty(kernels.attention_decode_scratch_floats(n, c["hq"], c["hd"], c["splits"]), device=DEV)
        kernels.attention_decode(q, want, k, v, table, table.shape[1], ctx_len, n, c["hq"], c["hkv"], c["hd"], 0.3,
                                 window=c["window"], n_splits=c["splits"], scratch=scratch, max_ctx=max(c["lengths"]),
                                 merge_in_scratch=True)
        got = torch.full_like(want, float("nan"))
        torch.cuda.synchronize()
        before = (device_free_bytes(), torch.cuda.memory_reserved())
        rc = call_static(lib, q, k, v, table, ctx_len, got, c["hq"], c["hkv"], c["hd"], 0.3, c["window"], c["splits"])
        assert rc == 0, lib.bt_last_error().decode()
        torch.cuda.synchronize()
        assert (device_free_bytes(), torch.cuda.memory_reserved()) == before, "the call took device memory"
        err = float((got.double() - want.double()).abs().max() / want.double().abs().max())
        assert err <= tol, f"{c}: {err:.3e}"
        # ... and both give what the formula gives
        plain = plain_attention(q, k, v, table, c["lengths"], c["hq"], c["hkv"], c["hd"], 0.3, c["window"])
        err = float((got.double().cpu() - plain).abs().max() / plain.abs().max())
        assert err <= max(tol, 1e-5) * (4 if dtype == torch.bfloat16 else 1), f"{c} against the formula: {err:.3e}"
        status = c_int(-1)
        assert lib.bt_attention_decode_static_status(ctypes.byref(status)) == 0 and status.value == 0


def test_static_scratch_entry_point_over_a_ring_of_pages():
    """A windowed layer's table is a ring: table_len pages that positions cycle through (table_len < the pages a
    full context would need).  Window 100 over a ring of 3 pages, contexts past the ring's first turn."""
    lib = kernels.library()
    lib.bt_attention_decode_static.restype = c_int
    lengths, hq, hkv, hd, window, ring = [450, 131, 193], 4, 2, 32, 100, 3
    g = torch.Generator().manual_seed(9)
    n = len(lengths)
    table = torch.randperm(n * ring, generator=g).view(n, ring).to(torch.int32).to(DEV)
    k = torch.randn(n * ring, hkv, PAGE, hd, generator=g).to(DEV)
    v = torch.randn(n * ring, hkv, PAGE, hd, generator=g).to(DEV)
    q = torch.randn(n, hq * hd, generator=g).to(DEV)
    ctx_len = torch.tensor(lengths, dtype=torch.int32, device=DEV)
    got = torch.full((n, hq * hd), float("nan"), device=DEV)
    rc = call_static(lib, q, k, v, table, ctx_len, got, hq, hkv, hd, 0.2, window, 2, table_len=ring)
    assert rc == 0, lib.bt_last_error().decode()
    torch.cuda.synchronize()
    plain = plain_attention(q, k, v, table, lengths, hq, hkv, hd, 0.2, window, table_len=ring)
    assert float((got.double().cpu() - plain).abs().max() / plain.abs().max()) < 1e-5


def test_static_scratch_entry_point_takes_an_empty_sequence():
    """A sequence of length 0 (an empty or finished request that still rides in the batch) yields zeros and
    touches no page."""
    lib = kernels.library()
    lib.bt_attention_decode_static.restype = c_int
    lengths, hq, hd = [70, 0, 5], 2, 16
    k, v, table = paged([70, 1, 5], hq, hd, torch.float32, 4)
    q = torch.randn(3, hq * hd, generator=torch.Generator().manual_seed(4)).to(DEV)
    ctx_len = torch.tensor(lengths, dtype=torch.int32, device=DEV)
    got = torch.full((3, hq * hd), float("nan"), device=DEV)
    assert call_static(lib, q, k, v, table, ctx_len, got, hq, hq, hd, 0.5, 0, 2) == 0, lib.bt_last_error().decode()
    torch.cuda.synchronize()
    plain = plain_attention(q, k, v, table, lengths, hq, hq, hd, 0.5, 0)
    assert float(got[1].abs().max()) == 0.0
    assert float((got.double().cpu() - plain).abs().max()) < 1e-5


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    lib = kernels.library()
    lib.bt_attention_decode_static.restype = c_int
    n, hq, hd, splits = 64, 64, 128, 2                     # 64 * 64 * 2 * 130 floats > 2^20
    assert n * hq * splits * (hd + 2) > STATIC_FLOATS
    k, v, table = paged([10] * n, 1, hd, torch.bfloat16, 3)
    q = torch.zeros(n, hq * hd, device=DEV, dtype=torch.bfloat16)
    out = torch.zeros_like(q)
    ctx_len = torch.full((n,), 10, dtype=torch.int32, device=DEV)
    rc = call_static(lib, q, k, v, table, ctx_len, out, hq, 1, hd, 1.0, 0, splits)
    message = lib.bt_last_error().decode()
    assert rc != 0 and "exceed the built-in" in message and str(STATIC_FLOATS) in message
    # more (sequence, head) pairs than the built-in merge tickets (16384), though the scratch would do
    n, hq, hd = 300, 64, 8
    assert n * hq > 16384 and n * hq * 2 * (hd + 2) <= STATIC_FLOATS
    k, v, table = paged([3] * n, 1, hd, torch.bfloat16, 5)
    q = torch.zeros(n, hq * hd, device=DEV, dtype=torch.bfloat16)
    out = torch.zeros_like(q)
    ctx_len = torch.full((n,), 3, dtype=torch.int32, device=DEV)
    rc = call_static(lib, q, k, v, table, ctx_len, out, hq, 1, hd, 1.0, 0, 2)
    assert rc != 0 and "merge tickets" in lib.bt_last_error().decode()
    # sizes out of range are refused before any product is formed
    rc = call_static(lib, q, k, v, table, ctx_len, out, 70000, 1, hd, 1.0, 0, 2)
    assert rc != 0 and "out of range" in lib.bt_last_error().decode()
    torch.cuda.synchronize()
