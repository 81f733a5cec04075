"""Each CUDA kernel alone against a plain float64 formula, at sizes other than the engine's."""
import math

import numpy as np
import pytest
import torch

import plain_gpt2 as plain
from burn_transformers_b200 import kernels
from burn_transformers_b200.errors import KernelError, ShapeError

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = kernels.PAGE_SIZE
# a kernel's own error: 32-bit sums of a few hundred terms; bfloat16 outputs are rounded to 8 bits once
TOL = {torch.float32: 2e-6, torch.bfloat16: 4e-3}


def rel(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(1234)


def test_library_is_the_built_one():
    lib = kernels.library()
    assert lib.bt_abi_version() == 1
    with pytest.raises(KernelError, match="CUDA device only"):
        kernels.layernorm(torch.zeros(2, 8), torch.ones(8), None, torch.zeros(2, 8), 1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width, vocab, n_pos", [(40, 33, 17), (1000, 129, 70)])
def test_embed(dtype, width, vocab, n_pos):
    wte = torch.randn(vocab, width, device=DEV).to(dtype)
    wpe = torch.randn(n_pos, width, device=DEV).to(dtype)
    tok = torch.randint(0, vocab, (23,), device=DEV, dtype=torch.int32)
    pos = torch.randint(0, n_pos, (23,), device=DEV, dtype=torch.int32)
    out = torch.empty(23, width, device=DEV)
    kernels.embed(tok, pos, wte, wpe, out)
    assert rel(out, wte.double()[tok.long()] + wpe.double()[pos.long()]) < 2e-7   # one 32-bit add
    kernels.embed(tok, pos, wte, None, out)
    assert torch.equal(out, wte.float()[tok.long()])
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    tok[5] = vocab
    kernels.embed(tok, pos, wte, wpe, out, status=status)
    assert int(status) == 6 and float(out[5].abs().max()) == 0.0     # reported, nothing read outside the table


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width, eps", [(24, 1e-5), (770, 1e-6), (4099, 1e-3)])
def test_layernorm(out_dtype, width, eps):
    x = torch.randn(13, width, device=DEV) * 5 + 100.0        # a large mean: E[x^2]-E[x]^2 would lose it
    g, b = torch.randn(width, device=DEV), torch.randn(width, device=DEV)
    out = torch.empty(13, width, device=DEV, dtype=out_dtype)
    kernels.layernorm(x, g, b, out, eps)
    want = torch.nn.functional.layer_norm(x.double(), (width,), g.double(), b.double(), eps)
    assert rel(out, want) < (1e-5 if out_dtype == torch.float32 else 4e-3)
    rows = torch.tensor([12, 0, 0, 7], dtype=torch.int32, device=DEV)
    picked = torch.empty(4, width, device=DEV, dtype=out_dtype)
    kernels.layernorm(x, g, None, picked, eps, rows=rows)
    want = torch.nn.functional.layer_norm(x.double()[rows.long()], (width,), g.double(), None, eps)
    assert rel(picked, want) < (1e-5 if out_dtype == torch.float32 else 4e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m, n, k", [(1, 50, 24), (7, 777, 240), (65, 64, 17), (200, 130, 1000)])
@pytest.mark.parametrize("nk", [False, True])
def test_linear_simt(dtype, m, n, k, nk):
    a = torch.randn(m, k, device=DEV).to(dtype)
    w = torch.randn(k, n, device=DEV).to(dtype)
    bias, res = torch.randn(n, device=DEV), torch.randn(m, n, device=DEV)
    w_arg = w.t().contiguous() if nk else w
    plain_product = a.double() @ w.double()
    out = torch.empty(m, n, device=DEV)
    kernels.linear_simt(a, w_arg, None, out, w_is_nk=nk)
    assert rel(out, plain_product) < 2e-6
    for act, fn in (("gelu_new", lambda t: torch.nn.functional.gelu(t, approximate="tanh")),
                    ("gelu", torch.nn.functional.gelu)):
        out = res.clone()
        kernels.linear_simt(a, w_arg, bias, out, w_is_nk=nk, activation=act, residual=out)     # in place
        assert rel(out, fn(plain_product + bias.double()) + res.double()) < 2e-6
    if dtype == torch.bfloat16:
        low = torch.empty(m, n, device=DEV, dtype=dtype)
        kernels.linear_simt(a, w_arg, bias, low, w_is_nk=nk)
        assert rel(low, plain_product + bias.double()) < 4e-3
    # rows beyond m are not touched
    big = torch.full((m + 3, n), 7.0, device=DEV)
    kernels.linear_simt(a, w_arg, None, big, m=m, w_is_nk=nk)
    assert float((big[m:] - 7.0).abs().max()) == 0.0
    with pytest.raises(ShapeError):
        kernels.linear_simt(a, w_arg, None, torch.empty(m, n + 1, device=DEV), w_is_nk=nk)


@pytest.mark.parametrize("m", [1, 8, 16, 17, 64])
@pytest.mark.parametrize("n, k, nk, split", [(768, 768, False, 0), (2304, 768, False, 1), (768, 3072, False, 8),
                                             (104, 240, False, 4), (200, 96, False, 0), (1000, 96, True, 0),
                                             (777, 240, True, 2), (50257, 64, True, 0)])
def test_linear_skinny(m, n, k, nk, split):
    a = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(k, n, device=DEV) * 0.1).to(torch.bfloat16)
    w_arg = w.t().contiguous() if nk else w
    bias, res = torch.randn(n, device=DEV), torch.randn(m, n, device=DEV)
    assert kernels.linear_skinny_supports(m, n, k, nk, False)
    product = a.double() @ w.double()
    out = res.clone()
    kernels.linear_skinny(a, w_arg, bias, out, m=m, w_is_nk=nk, activation="gelu_new", residual=out, split=split)
    want = torch.nn.functional.gelu(product + bias.double(), approximate="tanh") + res.double()
    assert rel(out, want) < 2e-6
    low = torch.full((m + 2, n), 3.0, device=DEV, dtype=torch.bfloat16)
    kernels.linear_skinny(a, w_arg, None, low, m=m, w_is_nk=nk, split=split)
    assert rel(low[:m], product) < 4e-3 and float((low[m:].float() - 3.0).abs().max()) == 0.0
    # the same rows give the same result whatever else is in the call
    if m > 1:
        alone = torch.empty(1, n, device=DEV)
        both = torch.empty(m, n, device=DEV)
        kernels.linear_skinny(a[m - 1:].contiguous(), w_arg, bias, alone, m=1, w_is_nk=nk, split=split)
        kernels.linear_skinny(a, w_arg, bias, both, m=m, w_is_nk=nk, split=split)
        assert torch.equal(alone[0], both[m - 1])
    # LayerNorm of 32-bit rows on the way in, rows picked by an index
    if m <= 16 and kernels.linear_skinny_supports(m, n, k, nk, True):
        x = torch.randn(m + 3, k, device=DEV) * 2 + 3
        g, b = torch.randn(k, device=DEV), torch.randn(k, device=DEV)
        rows = torch.randperm(m + 3, device=DEV)[:m].to(torch.int32)
        normed = torch.nn.functional.layer_norm(x.double()[rows.long()], (k,), g.double(), b.double(), 1e-5)
        normed = normed.float().to(torch.bfloat16).double()          # the kernel rounds the rows once too
        out = torch.empty(m, n, device=DEV)
        kernels.linear_skinny(None, w_arg, bias, out, m=m, w_is_nk=nk, norm=(x, g, b, 1e-5, rows), split=split)
        assert rel(out, normed @ w.double() + bias.double()) < 2e-3   # a row value at a rounding tie may flip


@pytest.mark.parametrize("m", [1, 8, 9, 16, 17, 64])
@pytest.mark.parametrize("n, k, warps_k", [(768, 768, 0), (2304, 768, 4), (768, 3072, 2), (104, 240, 1), (203, 96, 4),
                                           (777, 200, 0), (50257, 64, 0)])
def test_linear_stream(m, n, k, warps_k):
    a = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) * 0.1).to(torch.bfloat16)
    bias, res = torch.randn(n, device=DEV), torch.randn(m, n, device=DEV)
    assert kernels.linear_stream_supports(m, n, k, False)
    product = a.double() @ w.double().T
    out = res.clone()
    kernels.linear_stream(a, w, bias, out, m=m, activation="gelu_new", residual=out, warps_k=warps_k)
    want = torch.nn.functional.gelu(product + bias.double(), approximate="tanh") + res.double()
    assert rel(out, want) < 2e-6
    low = torch.full((m + 2, n), 3.0, device=DEV, dtype=torch.bfloat16)
    kernels.linear_stream(a, w, None, low, m=m, activation="gelu", warps_k=warps_k)
    assert rel(low[:m], torch.nn.functional.gelu(product)) < 4e-3 and float((low[m:].float() - 3.0).abs().max()) == 0.0
    if m > 1:     # the same row gives the same bits whatever else is in the call
        alone, both = torch.empty(1, n, device=DEV), torch.empty(m, n, device=DEV)
        kernels.linear_stream(a[m - 1:].contiguous(), w, bias, alone, m=1, warps_k=warps_k)
        kernels.linear_stream(a, w, bias, both, m=m, warps_k=warps_k)
        assert torch.equal(alone[0], both[m - 1])
    if m <= 16:   # LayerNorm of 32-bit rows on the way in, rows picked by an index
        x = torch.randn(m + 3, k, device=DEV) * 2 + 3
        g, b = torch.randn(k, device=DEV), torch.randn(k, device=DEV)
        rows = torch.randperm(m + 3, device=DEV)[:m].to(torch.int32)
        normed = torch.nn.functional.layer_norm(x.double()[rows.long()], (k,), g.double(), b.double(), 1e-5)
        normed = normed.float().to(torch.bfloat16).double()          # the kernel rounds the rows once too
        out = torch.empty(m, n, device=DEV)
        kernels.linear_stream(None, w, bias, out, m=m, norm=(x, g, b, 1e-5, rows), warps_k=warps_k)
        assert rel(out, normed @ w.double().T + bias.double()) < 2e-3   # a row value at a rounding tie may flip
        out2 = torch.empty(m, n, device=DEV)
        kernels.linear_stream(None, w, None, out2, m=m, norm=(x, g, None, 1e-5, None), warps_k=warps_k)
        normed = torch.nn.functional.layer_norm(x.double()[:m], (k,), g.double(), None, 1e-5).float().to(torch.bfloat16)
        assert rel(out2, normed.double() @ w.double().T) < 2e-3


@pytest.mark.parametrize("m, n, k", [(128, 128, 64), (2048, 2304, 768), (300, 768, 3072), (1000, 3072, 768), (65, 200, 96),
                                     (129, 50257, 64), (2, 8, 8), (513, 776, 1000), (2048, 768, 768), (1900, 3000, 136)])
def test_linear_tcgen05(m, n, k):
    a = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) * 0.1).to(torch.bfloat16)
    bias, res = torch.randn(n, device=DEV), torch.randn(m, n, device=DEV)
    assert kernels.linear_tcgen05_supports(m, n, k)
    product = a.double() @ w.double().T
    # a 32-bit sum of K products: roundings add up like a random walk, sqrt(K) * 2^-24, with a factor for the
    # tensor core's own accumulation order
    tol = 4.0 * math.sqrt(k) * 2.0 ** -24
    out = torch.full((m + 1, n), 5.0, device=DEV)
    kernels.linear_tcgen05(a, w, None, out, m=m)
    assert rel(out[:m], product) < tol and float((out[m:] - 5.0).abs().max()) == 0.0
    out = res.clone()
    kernels.linear_tcgen05(a, w, bias, out, m=m, activation="gelu_new", residual=out)
    want = torch.nn.functional.gelu(product + bias.double(), approximate="tanh") + res.double()
    assert rel(out, want) < tol
    low = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    kernels.linear_tcgen05(a, w, bias, low, m=m, activation="gelu")
    assert rel(low, torch.nn.functional.gelu(product + bias.double())) < 4e-3
    assert int(kernels.kernel_status(a.device)) == 0


@pytest.mark.parametrize("m", [17, 33, 64])
@pytest.mark.parametrize("n, k", [(768, 768), (2304, 768), (768, 3072), (104, 240), (200, 96), (777, 1600), (1000, 72),
                                  (64, 4096), (8237, 136)])
def test_linear_mid(m, n, k):
    """The product for 17 to 64 rows: sizes that are no multiples of its tiles, K longer than its ring of stages."""
    a = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) * 0.1).to(torch.bfloat16)
    bias, res = torch.randn(n, device=DEV), torch.randn(m, n, device=DEV)
    assert kernels.linear_mid_supports(m, n, k)
    product = a.double() @ w.double().T
    out = res.clone()
    kernels.linear_mid(a, w, bias, out, m=m, activation="gelu_new", residual=out)
    want = torch.nn.functional.gelu(product + bias.double(), approximate="tanh") + res.double()
    assert rel(out, want) < 4 * math.sqrt(k) * 2.0 ** -24 + 1e-6
    low = torch.full((m + 2, n), 3.0, device=DEV, dtype=torch.bfloat16)
    kernels.linear_mid(a, w, None, low, m=m)
    assert rel(low[:m], product) < 4e-3 and float((low[m:].float() - 3.0).abs().max()) == 0.0
    # the same rows give the same result whatever else is in the call
    alone = torch.empty(1, n, device=DEV)
    both = torch.empty(m, n, device=DEV)
    kernels.linear_mid(a[m - 1:].contiguous(), w, bias, alone, m=1)
    kernels.linear_mid(a, w, bias, both, m=m)
    assert torch.equal(alone[0], both[m - 1])
    assert int(kernels.kernel_status(a.device)) == 0


@pytest.mark.parametrize("split", [1, 2, 4, 8])
@pytest.mark.parametrize("n, k", [(768, 3072), (1000, 72), (52, 1608)])
def test_linear_mid_split_over_a_cluster(n, k, split):
    """K cut over the blocks of a cluster (slices that end inside a stage, members without any k) gives the whole
    sum, the same at every call."""
    m = 41
    a = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) * 0.1).to(torch.bfloat16)
    bias, res = torch.randn(n, device=DEV), torch.randn(m, n, device=DEV)
    want = torch.nn.functional.gelu(a.double() @ w.double().T + bias.double(), approximate="tanh") + res.double()
    outs = []
    for _ in range(2):
        out = res.clone()
        kernels.linear_mid(a, w, bias, out, m=m, activation="gelu_new", residual=out, split=split)
        outs.append(out)
    assert rel(outs[0], want) < 4 * math.sqrt(k) * 2.0 ** -24 + 1e-6
    assert torch.equal(outs[0], outs[1])
    assert int(kernels.kernel_status(a.device)) == 0


def test_linear_mid_refuses_what_it_cannot_do():
    assert not kernels.linear_mid_supports(65, 64, 64)
    assert not kernels.linear_mid_supports(20, 64, 100)          # rows of 100 bfloat16 are not 16-byte chunks
    with pytest.raises(KernelError, match="not supported"):
        kernels.linear_mid(torch.zeros(20, 100, device=DEV, dtype=torch.bfloat16),
                           torch.zeros(64, 100, device=DEV, dtype=torch.bfloat16), None, torch.zeros(20, 64, device=DEV), m=20)
    with pytest.raises(KernelError, match="split"):
        kernels.linear_mid(torch.zeros(20, 64, device=DEV, dtype=torch.bfloat16),
                           torch.zeros(64, 64, device=DEV, dtype=torch.bfloat16), None, torch.zeros(20, 64, device=DEV), m=20,
                           split=3)


@pytest.mark.parametrize("m", [1, 17, 64, 100, 128])
@pytest.mark.parametrize("n, k", [(256, 128), (768, 3072), (200, 72), (130, 64), (1000, 520), (1604, 6400), (2304, 776)])
def test_linear_few_tcgen05(m, n, k):
    """The tcgen05 product with the weights on the tensor cores' M side: column tiles that end inside a tile, rows
    that are no multiple of 16, K that ends inside a stage and is longer than the ring, the split the library
    chooses."""
    a = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) * 0.1).to(torch.bfloat16)
    bias, res = torch.randn(n, device=DEV), torch.randn(m, n, device=DEV)
    assert kernels.linear_few_tcgen05_supports(m, n, k)
    product = a.double() @ w.double().T
    out = torch.full((m + 2, n), 3.0, device=DEV)
    out[:m] = res
    kernels.linear_few_tcgen05(a, w, bias, out, m=m, activation="gelu_new", residual=out)
    want = torch.nn.functional.gelu(product + bias.double(), approximate="tanh") + res.double()
    assert rel(out[:m], want) < 4 * math.sqrt(k) * 2.0 ** -24 + 1e-6 and float((out[m:] - 3.0).abs().max()) == 0.0
    low = torch.full((m + 2, n), 3.0, device=DEV, dtype=torch.bfloat16)
    kernels.linear_few_tcgen05(a, w, None, low, m=m)
    assert rel(low[:m], product) < 4e-3 and float((low[m:].float() - 3.0).abs().max()) == 0.0
    low = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    kernels.linear_few_tcgen05(a, w, bias, low, m=m, activation="gelu")
    assert rel(low, torch.nn.functional.gelu(product + bias.double())) < 4e-3
    # the same rows give the same result whatever else is in the call
    alone = torch.empty(1, n, device=DEV)
    both = torch.empty(m, n, device=DEV)
    kernels.linear_few_tcgen05(a[m - 1:].contiguous(), w, bias, alone, m=1)
    kernels.linear_few_tcgen05(a, w, bias, both, m=m)
    assert torch.equal(alone[0], both[m - 1])
    assert int(kernels.kernel_status(a.device)) == 0


@pytest.mark.parametrize("split", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("n, k", [(768, 3072), (300, 520), (52, 1608)])
def test_linear_few_tcgen05_split_over_a_cluster(n, k, split):
    """K cut over the blocks of a cluster (slices that end inside a stage) gives the whole sum, the same at every
    call; a split that would leave a block without any k is refused."""
    m = 41
    a = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) * 0.1).to(torch.bfloat16)
    bias, res = torch.randn(n, device=DEV), torch.randn(m, n, device=DEV)
    k_blocks = -(-k // 64)
    if (split - 1) * -(-k_blocks // split) >= k_blocks:
        with pytest.raises(KernelError, match="without any of K"):
            kernels.linear_few_tcgen05(a, w, bias, res.clone(), m=m, split=split)
        return
    want = torch.nn.functional.gelu(a.double() @ w.double().T + bias.double(), approximate="tanh") + res.double()
    outs = []
    for _ in range(2):
        out = res.clone()
        kernels.linear_few_tcgen05(a, w, bias, out, m=m, activation="gelu_new", residual=out, split=split)
        outs.append(out)
    assert rel(outs[0], want) < 4 * math.sqrt(k) * 2.0 ** -24 + 1e-6
    assert torch.equal(outs[0], outs[1])
    assert int(kernels.kernel_status(a.device)) == 0


def test_linear_few_tcgen05_refuses_what_it_cannot_do():
    assert not kernels.linear_few_tcgen05_supports(129, 64, 64)
    assert not kernels.linear_few_tcgen05_supports(20, 64, 100)          # rows of 100 bfloat16 are not 16-byte chunks
    with pytest.raises(KernelError, match="not supported"):
        kernels.linear_few_tcgen05(torch.zeros(20, 100, device=DEV, dtype=torch.bfloat16),
                                   torch.zeros(64, 100, device=DEV, dtype=torch.bfloat16), None, torch.zeros(20, 64, device=DEV),
                                   m=20)
    with pytest.raises(KernelError, match="split"):
        kernels.linear_few_tcgen05(torch.zeros(20, 64, device=DEV, dtype=torch.bfloat16),
                                   torch.zeros(64, 64, device=DEV, dtype=torch.bfloat16), None, torch.zeros(20, 64, device=DEV),
                                   m=20, split=9)


def test_linear_skinny_refuses_what_it_cannot_do():
    assert not kernels.linear_skinny_supports(65, 64, 64, False, False)
    assert not kernels.linear_skinny_supports(4, 100, 64, False, False)     # [K,N] rows of 100 are not 16-byte chunks
    assert not kernels.linear_skinny_supports(4, 64, 100, True, False)
    assert not kernels.linear_skinny_supports(17, 64, 64, False, True)      # the fused LayerNorm takes one 16-row tile
    with pytest.raises(KernelError, match="not supported"):
        kernels.linear_skinny(torch.zeros(4, 100, device=DEV, dtype=torch.bfloat16),
                              torch.zeros(100, 100, device=DEV, dtype=torch.bfloat16), None,
                              torch.zeros(4, 100, device=DEV), m=4)


# ---- attention ---------------------------------------------------------------------------------

def make_paged(lengths, n_kv_heads, head_dim, dtype, table_len=None, extra_pages=3):
    """Random keys and values in shuffled pages.  Returns pools, table and the dense [seq][pos] copies."""
    n = len(lengths)
    width = max(-(-max(lengths) // PAGE), 1) if table_len is None else table_len
    n_pages = n * width + extra_pages
    order = torch.randperm(n_pages).tolist()
    table = torch.zeros(n, width, dtype=torch.int32)
    k_pool = torch.randn(n_pages, n_kv_heads, PAGE, head_dim).to(dtype)
    v_pool = torch.randn(n_pages, n_kv_heads, PAGE, head_dim).to(dtype)
    for s in range(n):
        for i in range(width):
            table[s, i] = order.pop()
    dense_k, dense_v = [], []
    for s, length in enumerate(lengths):
        pos = torch.arange(length)
        pages = table[s, (pos // PAGE) % width].long()
        dense_k.append(k_pool[pages, :, pos % PAGE].double())      # [L, H, hd]
        dense_v.append(v_pool[pages, :, pos % PAGE].double())
    return k_pool.to(DEV), v_pool.to(DEV), table.to(DEV), dense_k, dense_v


def attend(q, k, v, scale, q_pos, window=0, causal=True):
    """q: [Q, Hq, hd]; k, v: [L, Hkv, hd] float64; q_pos: position of each query."""
    hq, hkv = q.shape[1], k.shape[1]
    out = torch.zeros_like(q)
    pos = torch.arange(k.shape[0])
    for h in range(hq):
        s = (q[:, h] @ k[:, h // (hq // hkv)].T) * scale
        hidden = torch.zeros_like(s, dtype=torch.bool)
        if causal:
            hidden |= pos[None, :] > q_pos[:, None]
        if window:
            hidden |= pos[None, :] <= q_pos[:, None] - window
        s = s.masked_fill(hidden, -math.inf)
        p = torch.softmax(s, dim=-1).nan_to_num(0.0)
        out[:, h] = p @ v[:, h // (hq // hkv)]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hq, hkv, hd, window, splits", [
    (4, 4, 16, 0, 1), (5, 5, 48, 0, 3), (6, 2, 80, 0, 2), (8, 1, 128, 100, 4), (2, 2, 256, 0, 1), (3, 3, 32, 64, 7),
    (2, 2, 64, 0, 8), (2, 1, 64, 0, 12), (2, 2, 256, 0, 2)])
def test_attention_decode(dtype, hq, hkv, hd, window, splits):
    lengths = [1, 63, 64, 65, 300, 129] + ([1500] if hd == 256 else [])     # 1500 x 256 needs several rounds of pages
    k_pool, v_pool, table, dk, dv = make_paged(lengths, hkv, hd, dtype)
    n = len(lengths)
    q = torch.randn(n, (hq + 2 * hkv) * hd, device=DEV).to(dtype)     # queries inside a wider projection row
    ctx_len = torch.tensor(lengths, dtype=torch.int32, device=DEV)
    out = torch.empty(n, hq * hd, device=DEV, dtype=dtype)
    scratch = torch.empty(max(1, kernels.attention_decode_scratch_floats(n, hq, hd, splits)), device=DEV)
    scale = 0.37
    # (bfloat16 runs on tensor cores where the head size allows it, and on the multiply-add kernel when told so)
    for in_scratch, tensor_cores in ((False, True), (True, True), (False, False), (True, False)):
        if not tensor_cores and dtype == torch.float32:
            continue
        out.fill_(float("nan"))
        kernels.attention_decode(q, out, k_pool, v_pool, table, table.shape[1], ctx_len, n, hq, hkv, hd, scale,
                                 window=window, n_splits=splits, scratch=scratch, max_ctx=max(lengths),
                                 merge_in_scratch=in_scratch, tensor_cores=tensor_cores)
        for s, length in enumerate(lengths):
            qs = q[s, :hq * hd].double().cpu().view(1, hq, hd)
            want = attend(qs, dk[s], dv[s], scale, torch.tensor([length - 1]), window)
            assert rel(out[s].view(1, hq, hd), want) < TOL[dtype] * 2, f"sequence {s} of length {length}"
    assert int(kernels.kernel_status(q.device)) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("target", [0, 63, 64, 437, 699])
@pytest.mark.parametrize("splits", [1, 5])
def test_attention_decode_finds_one_far_key_among_hundreds(dtype, target, splits):
    """With near-uniform random scores a lost key changes the result by 1/700, less than a bfloat16 rounding.
    Here one key matches the query and carries a value of its own, so losing it changes everything."""
    hq = hkv = 2
    hd, length = 64, 700
    k_pool, v_pool, table, dk, dv = make_paged([length], hkv, hd, dtype)
    q = torch.randn(1, hq * hd, device=DEV).to(dtype)
    page, row = int(table[0, target // PAGE]), target % PAGE
    for h in range(hq):
        k_pool[page, h, row] = (q[0, h * hd:(h + 1) * hd].float() * 4.0).to(dtype)      # score ~ 4 |q|^2 >> the rest
        v_pool[page, h, row] = 50.0 + h
    ctx_len = torch.tensor([length], dtype=torch.int32, device=DEV)
    out = torch.empty(1, hq * hd, device=DEV, dtype=dtype)
    scratch = torch.empty(max(1, kernels.attention_decode_scratch_floats(1, hq, hd, splits)), device=DEV)
    kernels.attention_decode(q, out, k_pool, v_pool, table, table.shape[1], ctx_len, 1, hq, hkv, hd, 1.0,
                             n_splits=splits, scratch=scratch, max_ctx=length)
    got = out.float().view(hq, hd)
    for h in range(hq):
        assert float((got[h] - (50.0 + h)).abs().max()) < 0.5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_decode_window_edge(dtype):
    """The key just outside the window would win the softmax if it were seen; the key just inside must be seen."""
    hd, length, window = 32, 200, 70
    for inside in (True, False):
        k_pool, v_pool, table, _, _ = make_paged([length], 1, hd, dtype)
        q = torch.randn(1, hd, device=DEV).to(dtype)
        target = length - window if inside else length - window - 1
        page, row = int(table[0, target // PAGE]), target % PAGE
        k_pool[page, 0, row] = (q[0].float() * 4.0).to(dtype)
        v_pool[page, 0, row] = 90.0
        out = torch.empty(1, hd, device=DEV, dtype=dtype)
        scratch = torch.empty(kernels.attention_decode_scratch_floats(1, 1, hd, 2), device=DEV)
        kernels.attention_decode(q, out, k_pool, v_pool, table, table.shape[1],
                                 torch.tensor([length], dtype=torch.int32, device=DEV), 1, 1, 1, hd, 1.0,
                                 window=window, n_splits=2, scratch=scratch, max_ctx=length)
        assert (float(out.float().mean()) > 80.0) == inside


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hq, hkv, hd, window, causal", [
    (4, 4, 16, 0, True), (5, 5, 48, 0, True), (6, 3, 80, 0, True), (2, 1, 128, 40, True), (2, 2, 256, 0, True),
    (3, 3, 64, 0, False), (3, 3, 64, 0, True), (4, 2, 64, 70, True), (2, 2, 128, 0, True),
    # head sizes whose rows are no whole 16-byte pieces: copied and read element by element
    (3, 3, 4, 0, True), (2, 1, 7, 30, True), (5, 5, 20, 0, True), (2, 2, 1, 0, True), (2, 1, 100, 0, True)])
def test_attention_prefill_packed_and_paged(dtype, hq, hkv, hd, window, causal):
    """Several new tokens per sequence: from the step's own projections (sequences that start at 0) and from
    the pages (sequences that already hold tokens), with unequal lengths."""
    news, pasts = [1, 17, 64, 100, 200], [0, 0, 0, 0, 0]
    width = (hq + 2 * hkv) * hd
    n_tok = sum(news)
    proj = torch.randn(n_tok, width, device=DEV).to(dtype)
    seq_start = torch.tensor([0] + list(np.cumsum(news)), dtype=torch.int32, device=DEV)
    out = torch.empty(n_tok, hq * hd, device=DEV, dtype=dtype)
    scale = 0.3
    kernels.attention_prefill(proj, out, seq_start, torch.tensor(pasts, dtype=torch.int32, device=DEV),
                              len(news), max(news), hq, hkv, hd, scale, causal=causal, window=window,
                              k_offset=hq * hd, v_offset=(hq + hkv) * hd)
    p64 = proj.double().cpu()
    for s, n in enumerate(news):
        rows = p64[int(seq_start[s]):int(seq_start[s]) + n]
        q = rows[:, :hq * hd].view(n, hq, hd)
        k = rows[:, hq * hd:(hq + hkv) * hd].view(n, hkv, hd)
        v = rows[:, (hq + hkv) * hd:].view(n, hkv, hd)
        want = attend(q, k, v, scale, torch.arange(n), window, causal)
        got = out[int(seq_start[s]):int(seq_start[s]) + n].view(n, hq, hd)
        assert rel(got, want) < TOL[dtype] * 2, f"packed, sequence {s}"
    if not causal:
        return
    # paged: sequences hold `past` tokens already; the new tokens' keys are appended first
    pasts = [0, 5, 64, 130, 77]
    lengths = [p + n for p, n in zip(pasts, news)]
    k_pool, v_pool, table, dk, dv = make_paged(lengths, hkv, hd, dtype)
    positions = torch.cat([torch.arange(p, p + n) for p, n in zip(pasts, news)]).to(torch.int32).to(DEV)
    token_seq = torch.cat([torch.full((n,), s) for s, n in enumerate(news)]).to(torch.int32).to(DEV)
    ctx_len = torch.tensor(lengths, dtype=torch.int32, device=DEV)
    kernels.kv_append(proj, hq * hd, (hq + hkv) * hd, positions, token_seq, ctx_len, table, table.shape[1], k_pool,
                      v_pool, n_tok, hkv, hd)
    kernels.attention_prefill(proj, out, seq_start, torch.tensor(pasts, dtype=torch.int32, device=DEV),
                              len(news), max(news), hq, hkv, hd, scale, causal=True, window=window,
                              k_pool=k_pool, v_pool=v_pool, table=table, table_len=table.shape[1])
    for s, n in enumerate(news):
        rows = p64[int(seq_start[s]):int(seq_start[s]) + n]
        k = torch.cat([dk[s][:pasts[s]], rows[:, hq * hd:(hq + hkv) * hd].view(n, hkv, hd)])
        v = torch.cat([dv[s][:pasts[s]], rows[:, (hq + hkv) * hd:].view(n, hkv, hd)])
        want = attend(rows[:, :hq * hd].view(n, hq, hd), k, v, scale, torch.arange(pasts[s], pasts[s] + n), window)
        got = out[int(seq_start[s]):int(seq_start[s]) + n].view(n, hq, hd)
        assert rel(got, want) < TOL[dtype] * 2, f"paged, sequence {s}"


@pytest.mark.parametrize("impl", ["tcgen05"])
@pytest.mark.parametrize("hq, hkv, hd, window, causal", [(3, 3, 64, 0, True), (4, 2, 64, 150, True), (2, 1, 128, 0, True),
                                                         (2, 2, 128, 300, True), (2, 2, 64, 0, False)])
def test_attention_prefill_long_sequences_on_tensor_cores(impl, hq, hkv, hd, window, causal):
    """Both tensor-core kernels by name, over sequences of several key tiles (stages of the pipeline are used
    again), lengths at and beside the tile edges, packed and paged."""
    dtype = torch.bfloat16
    news = [700, 129, 128, 1, 257]
    width = (hq + 2 * hkv) * hd
    n_tok = sum(news)
    proj = torch.randn(n_tok, width, device=DEV).to(dtype)
    seq_start = torch.tensor([0] + list(np.cumsum(news)), dtype=torch.int32, device=DEV)
    out = torch.full((n_tok, hq * hd), 7.0, device=DEV, dtype=dtype)
    scale = 0.2
    kernels.attention_prefill(proj, out, seq_start, torch.zeros(len(news), dtype=torch.int32, device=DEV),
                              len(news), max(news), hq, hkv, hd, scale, causal=causal, window=window,
                              k_offset=hq * hd, v_offset=(hq + hkv) * hd, impl=impl)
    assert int(kernels.kernel_status(proj.device)) == 0
    p64 = proj.double().cpu()
    for s, n in enumerate(news):
        rows = p64[int(seq_start[s]):int(seq_start[s]) + n]
        q = rows[:, :hq * hd].view(n, hq, hd)
        k = rows[:, hq * hd:(hq + hkv) * hd].view(n, hkv, hd)
        v = rows[:, (hq + hkv) * hd:].view(n, hkv, hd)
        want = attend(q, k, v, scale, torch.arange(n), window, causal)
        got = out[int(seq_start[s]):int(seq_start[s]) + n].view(n, hq, hd)
        assert rel(got, want) < TOL[dtype] * 2, f"packed, sequence {s}"
    if not causal or window:
        return
    pasts = [100, 64, 3, 500, 0]
    lengths = [p + n for p, n in zip(pasts, news)]
    k_pool, v_pool, table, dk, dv = make_paged(lengths, hkv, hd, dtype)
    positions = torch.cat([torch.arange(p, p + n) for p, n in zip(pasts, news)]).to(torch.int32).to(DEV)
    token_seq = torch.cat([torch.full((n,), s) for s, n in enumerate(news)]).to(torch.int32).to(DEV)
    ctx_len = torch.tensor(lengths, dtype=torch.int32, device=DEV)
    kernels.kv_append(proj, hq * hd, (hq + hkv) * hd, positions, token_seq, ctx_len, table, table.shape[1], k_pool,
                      v_pool, n_tok, hkv, hd)
    out.fill_(7.0)
    kernels.attention_prefill(proj, out, seq_start, torch.tensor(pasts, dtype=torch.int32, device=DEV),
                              len(news), max(news), hq, hkv, hd, scale, causal=True, window=window,
                              k_pool=k_pool, v_pool=v_pool, table=table, table_len=table.shape[1], impl=impl)
    assert int(kernels.kernel_status(proj.device)) == 0
    for s, n in enumerate(news):
        rows = p64[int(seq_start[s]):int(seq_start[s]) + n]
        k = torch.cat([dk[s][:pasts[s]], rows[:, hq * hd:(hq + hkv) * hd].view(n, hkv, hd)])
        v = torch.cat([dv[s][:pasts[s]], rows[:, (hq + hkv) * hd:].view(n, hkv, hd)])
        want = attend(rows[:, :hq * hd].view(n, hq, hd), k, v, scale, torch.arange(pasts[s], pasts[s] + n), window)
        got = out[int(seq_start[s]):int(seq_start[s]) + n].view(n, hq, hd)
        assert rel(got, want) < TOL[dtype] * 2, f"paged, sequence {s}"


@pytest.mark.parametrize("impl", ["tcgen05"])
@pytest.mark.parametrize("hd", [64, 128])
def test_attention_prefill_far_key_future_key_and_window_edge(impl, hd):
    """One key among hundreds answers a late query: in another key tile far back it must be found, one position in
    the future it must not be seen, and with a window it is seen at the window's first position and not one before."""
    n, query = 600, 517
    base = (torch.randn(n, 3 * hd, device=DEV) * 0.05).to(torch.bfloat16)
    seq_start = torch.tensor([0, n], dtype=torch.int32, device=DEV)
    past = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.empty(n, hd, device=DEV, dtype=torch.bfloat16)

    def run(key, window):
        proj = base.clone()
        proj[query, :hd] = 2.0
        proj[key, hd:2 * hd] = 2.0
        proj[key, 2 * hd:] = 50.0
        kernels.attention_prefill(proj, out, seq_start, past, 1, n, 1, 1, hd, 1.0, window=window, k_offset=hd,
                                  v_offset=2 * hd, impl=impl)
        return out[query].float()

    assert float(run(3, 0).min()) > 45.0                       # far back, in the first key tile
    assert float(run(query, 0).min()) > 45.0                   # the query's own position
    assert float(run(query + 1, 0).abs().max()) < 2.0          # one position in the future
    window = 200
    assert float(run(query - window + 1, window).min()) > 45.0    # the window's first position
    assert float(run(query - window, window).abs().max()) < 2.0   # one before the window
    assert int(kernels.kernel_status(base.device)) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd", [32, 64])
def test_attention_prefill_never_looks_ahead(dtype, hd):
    """A future key that matches the query perfectly must not be seen; the same key in the past must."""
    n = 90
    proj = (torch.randn(n, 3 * hd, device=DEV) * 0.1).to(dtype)
    seq_start = torch.tensor([0, n], dtype=torch.int32, device=DEV)
    past = torch.zeros(1, dtype=torch.int32, device=DEV)
    query, key = 40, 41
    proj[query, :hd] = 3.0
    proj[key, hd:2 * hd] = 3.0
    proj[key, 2 * hd:] = 70.0
    out = torch.empty(n, hd, device=DEV, dtype=dtype)
    kernels.attention_prefill(proj, out, seq_start, past, 1, n, 1, 1, hd, 1.0, k_offset=hd, v_offset=2 * hd)
    assert float(out[query].float().abs().max()) < 5.0          # key 41 is in query 40's future
    proj[query + 2, :hd] = 3.0
    kernels.attention_prefill(proj, out, seq_start, past, 1, n, 1, 1, hd, 1.0, k_offset=hd, v_offset=2 * hd)
    assert float(out[query + 2].float().min()) > 60.0           # and in query 42's past


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hkv, hd", [(3, 16), (3, 4), (2, 7), (1, 1), (2, 100)])
def test_kv_append_pages_and_ring(dtype, hkv, hd):
    news, pasts = [70, 1], [60, 127]
    lengths = [p + n for p, n in zip(pasts, news)]
    n_tok = sum(news)
    proj = torch.randn(n_tok, 5 * hkv * hd, device=DEV).to(dtype)
    k_off, v_off = hkv * hd, 3 * hkv * hd
    positions = torch.cat([torch.arange(p, p + n) for p, n in zip(pasts, news)]).to(torch.int32).to(DEV)
    token_seq = torch.cat([torch.full((n,), s) for s, n in enumerate(news)]).to(torch.int32).to(DEV)
    ctx_len = torch.tensor(lengths, dtype=torch.int32, device=DEV)
    table = torch.tensor([[5, 2, 7], [1, 4, 0]], dtype=torch.int32, device=DEV)
    k_pool = torch.zeros(8, hkv, PAGE, hd, device=DEV, dtype=dtype)
    v_pool = torch.zeros_like(k_pool)
    kernels.kv_append(proj, k_off, v_off, positions, token_seq, ctx_len, table, 3, k_pool, v_pool, n_tok, hkv, hd)
    for t in range(n_tok):
        s, pos = int(token_seq[t]), int(positions[t])
        page = int(table[s, pos // PAGE])
        assert torch.equal(k_pool[page, :, pos % PAGE].reshape(-1), proj[t, k_off:k_off + hkv * hd])
        assert torch.equal(v_pool[page, :, pos % PAGE].reshape(-1), proj[t, v_off:v_off + hkv * hd])
    assert int((k_pool.float().abs().sum(dim=(1, 3)) > 0).sum()) == n_tok           # nothing else was written
    # a ring of one page keeps the last 64 positions only
    k_pool.zero_(); v_pool.zero_()
    kernels.kv_append(proj, k_off, v_off, positions, token_seq, ctx_len, table, 1, k_pool, v_pool, n_tok, hkv, hd)
    for t in range(n_tok):
        s, pos = int(token_seq[t]), int(positions[t])
        kept = pos >= lengths[s] - PAGE
        same = torch.equal(k_pool[int(table[s, 0]), :, pos % PAGE].reshape(-1), proj[t, k_off:k_off + hkv * hd])
        assert same == kept


# ---- selection ---------------------------------------------------------------------------------

def run_sample(logits, **kw):
    n = logits.shape[0]
    ids = torch.empty(n, dtype=torch.int32, device=DEV)
    logp = torch.empty(n, dtype=torch.float32, device=DEV)
    kernels.sample(logits, n, out_ids=ids, out_logp=logp, **kw)
    return ids.cpu().tolist(), logp.cpu().tolist()


@pytest.mark.parametrize("vocab", [19, 777, 50257])
def test_greedy_selection(vocab):
    z = torch.randn(5, vocab, device=DEV) * 3
    z[1, 7] = z[1, vocab - 1] = 50.0              # a tie: the lower index wins
    z[2, vocab - 1] = 60.0
    ids, logp = run_sample(z, do_sample=False)
    want = torch.log_softmax(z.double(), dim=-1)
    assert ids[1] == 7 and ids[2] == vocab - 1
    for r in range(5):
        assert ids[r] == int(torch.argmax(z[r]))
        assert abs(logp[r] - float(want[r, ids[r]])) < 1e-4


@pytest.mark.parametrize("vocab", [19, 1000, 50257])
@pytest.mark.parametrize("options", [dict(), dict(top_k=5), dict(top_p=0.7), dict(min_p=0.05),
                                     dict(top_k=40, top_p=0.9, min_p=0.01)])
def test_sampling_follows_the_inverse_cdf(vocab, options):
    temperature = 0.8
    if "top_k" in options:
        options = dict(options, top_k=min(options["top_k"], vocab - 1))
    row = (torch.randn(vocab) * 2.5).float()
    rows = 64
    z = row.repeat(rows, 1).contiguous().to(DEV)
    u = ((torch.arange(rows, dtype=torch.float64) + 0.5) / rows).float()
    u[0], u[-1] = 2.0 ** -24, 1 - 2.0 ** -24
    ids, logp = run_sample(z, do_sample=True, temperature=temperature, uniforms=u.to(DEV),
                           top_k=options.get("top_k", 0), top_p=options.get("top_p", 1.0), min_p=options.get("min_p", 0.0))
    processed = plain.process(row.double().numpy(), sample=True, temperature=temperature, **options)
    kept = np.isfinite(processed)
    assert all(kept[i] for i in ids), "a filtered token was drawn"
    assert ids[0] == int(np.argmax(kept)) and ids[-1] == int(len(kept) - 1 - np.argmax(kept[::-1]))
    e = np.where(kept, np.exp(processed - processed[kept].max()), 0.0)
    c = np.cumsum(e / e.sum())
    lsm = plain.log_softmax(np.where(kept, processed, -1e300))
    for r in range(rows):
        k = ids[r]
        below = c[k - 1] if k > 0 else 0.0
        assert below - 1e-5 <= float(u[r]) <= c[k] + 1e-5, f"row {r}: u={float(u[r])} outside [{below}, {c[k]}]"
        assert abs(logp[r] - lsm[k]) < 2e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_decode_files_the_new_token_itself(dtype):
    """Given the step's projections, the kernel reads the newest key and value from them and writes them into
    the page; the result equals appending first and attending then."""
    hq, hkv, hd = 6, 3, 32
    lengths = [1, 64, 65, 200]
    n = len(lengths)
    k_pool, v_pool, table, _, _ = make_paged(lengths, hkv, hd, dtype)
    proj = torch.randn(n, (hq + 2 * hkv) * hd, device=DEV).to(dtype)
    ctx_len = torch.tensor(lengths, dtype=torch.int32, device=DEV)
    k_ref, v_ref = k_pool.clone(), v_pool.clone()
    positions = (ctx_len - 1).contiguous()
    token_seq = torch.arange(n, dtype=torch.int32, device=DEV)
    kernels.kv_append(proj, hq * hd, (hq + hkv) * hd, positions, token_seq, ctx_len, table, table.shape[1], k_ref, v_ref,
                      n, hkv, hd)
    for splits in (1, 3):
        scratch = torch.empty(max(1, kernels.attention_decode_scratch_floats(n, hq, hd, splits)), device=DEV)
        want = torch.empty(n, hq * hd, device=DEV, dtype=dtype)
        kernels.attention_decode(proj, want, k_ref, v_ref, table, table.shape[1], ctx_len, n, hq, hkv, hd, 0.4,
                                 n_splits=splits, scratch=scratch, max_ctx=max(lengths))
        k_new, v_new = k_pool.clone(), v_pool.clone()
        got = torch.empty_like(want)
        kernels.attention_decode(proj, got, k_new, v_new, table, table.shape[1], ctx_len, n, hq, hkv, hd, 0.4,
                                 n_splits=splits, scratch=scratch, new_kv_offsets=(hq * hd, (hq + hkv) * hd),
                                 max_ctx=max(lengths))
        assert torch.equal(got, want)
        assert torch.equal(k_new, k_ref) and torch.equal(v_new, v_ref)


def test_logit_edits():
    z = torch.tensor([[1.0, -2.0, 3.0, 4.0, 0.5], [1.0, 1.0, 1.0, 1.0, 1.0]], device=DEV)
    rows = torch.tensor([0, 0, 0, 1], dtype=torch.int32, device=DEV)
    toks = torch.tensor([0, 1, 3, 4], dtype=torch.int32, device=DEV)
    vals = torch.tensor([0.5, 2.0, 0.25, 0.0,      # (1 + .5) / 2 - .25 = 0.5
                         0.0, 2.0, 0.0, 0.0,       # -2 * 2 = -4
                         0.0, 1.0, 0.0, 1.0,       # banned
                         1.0, 1.0, 3.0, 0.0], device=DEV)
    kernels.logit_edits(z, rows, toks, vals, 4)
    assert z.cpu().tolist() == [[0.5, -4.0, 3.0, -math.inf, 0.5], [1.0, 1.0, 1.0, 1.0, -1.0]]


@pytest.mark.parametrize("vocab", [777, 50257])
def test_a_uniform_next_to_one_selects_the_last_survivor_never_a_filtered_token(vocab):
    """The threshold u * total and the running sums round differently; with u a few units in the last place below 1 the
    count of sums below the threshold may run past the last token that survived the filters.  Whatever the rounding,
    the selected token must be one of the survivors: here the top 3 of each row, none of them the last index."""
    g = torch.Generator().manual_seed(vocab)
    z = (torch.randn(64, vocab, generator=g) * 2).to(DEV)
    z[:, vocab - 1] = -30.0                      # the token the count would end on is filtered out
    top = torch.topk(z, 3, dim=-1).indices.cpu()
    for u in (1.0 - 2.0 ** -24, 1.0 - 2.0 ** -23, 0.999999):
        uniforms = torch.full((64,), u, dtype=torch.float32, device=DEV)
        ids, logp = run_sample(z, do_sample=True, temperature=0.7, top_k=3, uniforms=uniforms)
        for r, token in enumerate(ids):
            assert token in top[r].tolist(), (u, r, token)
            assert token == int(top[r].max()), "the largest uniform selects the survivor with the largest index"
        assert all(np.isfinite(logp))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("splits, new_kv", [(1, False), (3, False), (2, True)])
def test_attention_decode_with_an_empty_sequence_in_the_batch(dtype, splits, new_kv):
    """ctx_len 0 (an empty or finished request that still rides in the batch): zeros for that row, no page touched
    (with `new_kv` the kernel would otherwise file a key at position -1), the other rows as usual."""
    hq, hkv, hd = 4, 2, 64
    lengths = [130, 0, 64]
    k_pool, v_pool, table, dk, dv = make_paged([130, 1, 64], hkv, hd, dtype)
    q = torch.randn(3, (hq + 2 * hkv) * hd, device=DEV).to(dtype)
    ctx_len = torch.tensor(lengths, dtype=torch.int32, device=DEV)
    pools_before = (k_pool.clone(), v_pool.clone())
    offsets = (hq * hd, (hq + hkv) * hd) if new_kv else None
    scratch = torch.empty(max(1, kernels.attention_decode_scratch_floats(3, hq, hd, splits)), device=DEV)
    for in_scratch, tensor_cores in ((False, True), (True, False)):
        out = torch.full((3, hq * hd), float("nan"), device=DEV, dtype=dtype)
        kernels.attention_decode(q, out, k_pool, v_pool, table, table.shape[1], ctx_len, 3, hq, hkv, hd, 0.2,
                                 n_splits=splits, scratch=scratch, max_ctx=130, merge_in_scratch=in_scratch,
                                 tensor_cores=tensor_cores, new_kv_offsets=offsets)
        torch.cuda.synchronize()
        assert float(out[1].float().abs().max()) == 0.0
        page = int(table[1, 0])
        assert torch.equal(k_pool[page], pools_before[0][page]) and torch.equal(v_pool[page], pools_before[1][page])
        for s in (0, 2):
            keys, values = dk[s].clone(), dv[s].clone()
            if new_kv:      # the newest key and value come from the projection row
                keys[-1] = q[s, offsets[0]:offsets[0] + hkv * hd].double().cpu().view(hkv, hd)
                values[-1] = q[s, offsets[1]:offsets[1] + hkv * hd].double().cpu().view(hkv, hd)
            want = attend(q[s, :hq * hd].double().cpu().view(1, hq, hd), keys, values, 0.2, torch.tensor([lengths[s] - 1]))
            assert rel(out[s].view(1, hq, hd), want) < TOL[dtype] * 2
    assert int(kernels.kernel_status(q.device)) == 0
