"""Self-attention over the cache."""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.spec import PAGE_SIZE, CacheNeed, KvSpec
from ..errors import CacheError, ShapeError
from ..weights.spec import MATRIX, VECTOR, TensorSpec
from .base import Mixer
from .linear import linear

_SM_COUNTS: dict = {}


def _sm_count(device) -> int:
    """Streaming multiprocessors of `device` (asked of the driver once)."""
    if device not in _SM_COUNTS:
        _SM_COUNTS[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return _SM_COUNTS[device]


class CausalSelfAttention(Mixer):
    """Multi-head (or grouped) attention with one fused query|key|value projection.

    [q|k|v] = x @ qkv.weight + qkv.bias with the weight stored [in, out]; head h owns channels
    h*head_dim..(h+1)*head_dim of its block; scores are (q . k) * scale, masked causally (and by
    `window` if given), softmax in 32-bit, then the value mix and the output projection, whose
    result is added to the residual stream (src/models/gpt2/model.rs:114-142, 218-261;
    src/attention/dispatch.rs:277-430 of the reference).  `n_kv_heads` < `n_heads` shares each key
    head among consecutive query heads.
    """

    accepts_lazy_norm = True
    linear_weights = ("qkv.weight", "out.weight")
    MAX_HEAD_DIM = 256      # every head size up to this runs (the kernels made for 16-byte pieces where they fit)

    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int, scale: float, *,
                 causal: bool = True, window: int | None = None, bias: bool = True,
                 init_std: float = 0.02, out_init_std: float | None = None, positions=None):
        if n_heads <= 0 or n_kv_heads <= 0 or n_heads % n_kv_heads:
            raise ShapeError(f"{n_heads} query heads cannot share {n_kv_heads} key heads")
        if not 1 <= head_dim <= self.MAX_HEAD_DIM:
            raise ShapeError(f"head_dim {head_dim} is outside 1..{self.MAX_HEAD_DIM}, the head sizes the attention "
                             f"kernels take")
        self.width, self.n_heads, self.n_kv_heads, self.head_dim = width, n_heads, n_kv_heads, head_dim
        self.scale, self.causal, self.window, self.has_bias = float(scale), causal, window, bias
        # a position encoding that rotates (parts.base.PositionEncoding.rotates): applied to the new queries and
        # keys before the keys are filed, so that the cache holds rotated keys
        self.positions = positions if positions is not None and positions.rotates else None
        self.q_width = n_heads * head_dim
        self.kv_width = n_kv_heads * head_dim
        self.proj_width = self.q_width + 2 * self.kv_width
        self.init_std = init_std
        self.out_init_std = init_std if out_init_std is None else out_init_std

    def specs(self):
        specs = {"qkv.weight": TensorSpec((self.width, self.proj_width), MATRIX, ("normal", self.init_std)),
                 "out.weight": TensorSpec((self.q_width, self.width), MATRIX, ("normal", self.out_init_std))}
        if self.has_bias:
            specs["qkv.bias"] = TensorSpec((self.proj_width,), VECTOR, ("zeros",))
            specs["out.bias"] = TensorSpec((self.width,), VECTOR, ("zeros",))
        return specs

    def cache_need(self):
        return CacheNeed(kv=KvSpec(self.n_kv_heads, self.head_dim, self.window))

    def _splits(self, ctx) -> int:
        """Blocks per (sequence, head) in a decode step: enough to fill the GPU about twice, none when the batch
        does that by itself (a split costs a merge); at most 8, so that they merge inside one thread-block
        cluster, and at most one per page."""
        units = max(1, ctx.n_seqs * self.n_heads)
        span = ctx.ctx_bound if self.window is None else min(ctx.ctx_bound, self.window)
        pages = max(1, -(-span // PAGE_SIZE))
        by_fill = -(-2 * _sm_count(ctx.ws.device) // units)
        return int(max(1, min(by_fill, pages, 8)))

    def forward(self, ctx, x, residual, entry, owns_cache=True):
        n = ctx.n_tokens
        dtype = ctx.dtype
        proj = ctx.ws.take((n, self.proj_width), dtype)
        linear(ctx, x, self.t_qkv_weight, self.t_qkv_bias if self.has_bias else None, proj, m=n,
               w_is_nk=self.nk_qkv_weight)
        program = getattr(ctx, "program", None)
        if self.positions is not None:
            if program is not None:
                from ..engine.program import ProgramUnsupported
                raise ProgramUnsupported("a rotating position encoding has no phase in the fused step")
            self.positions.rotate(ctx, proj, self.n_heads, self.n_kv_heads, self.head_dim)
        k_pool, v_pool, group, g = ctx.cache.layer_pools(entry)
        table = ctx.tables[g]
        window = self.window or 0
        if owns_cache and not ctx.is_decode:
            side = getattr(ctx, "side", None) if ctx.fresh else None
            if side is not None:
                # fresh sequences attend over the step's own projections: nothing in this step reads the pages, so
                # the keys and values are filed beside the attention, on the step's second stream
                side.fork()
                with side.stream_context():
                    kernels.kv_append(proj, self.q_width, self.q_width + self.kv_width, ctx.positions, ctx.token_seq,
                                      ctx.ctx_len, table, group.table_len, k_pool, v_pool, n, self.n_kv_heads, self.head_dim)
            else:
                kernels.kv_append(proj, self.q_width, self.q_width + self.kv_width, ctx.positions, ctx.token_seq,
                                  ctx.ctx_len, table, group.table_len, k_pool, v_pool, n, self.n_kv_heads, self.head_dim)
        if program is not None and ctx.is_decode:
            # recorded as a phase of the fused step; its partial results are merged by the output projection
            mixed = program.add_attention(ctx, proj, k_pool, v_pool, table, group.table_len, n_heads=self.n_heads,
                                          n_kv_heads=self.n_kv_heads, head_dim=self.head_dim, scale=self.scale,
                                          window=window,
                                          new_kv_offsets=(self.q_width, self.q_width + self.kv_width) if owns_cache else None)
            linear(ctx, mixed, self.t_out_weight, self.t_out_bias if self.has_bias else None, residual, m=n,
                   residual=residual, w_is_nk=self.nk_out_weight)
            return
        mixed = ctx.ws.take((n, self.q_width), dtype)
        if ctx.is_decode and not kernels.attention_decode_supports(self.head_dim, proj.shape[1], dtype):
            # a head size whose rows are no whole 16-byte pieces: the step's keys and values are filed first, then
            # the kernel that reads element by element attends over the pages (one new token per sequence)
            kernels.kv_append(proj, self.q_width, self.q_width + self.kv_width, ctx.positions, ctx.token_seq,
                              ctx.ctx_len, table, group.table_len, k_pool, v_pool, n, self.n_kv_heads, self.head_dim)
            kernels.attention_prefill(proj, mixed, ctx.seq_start, ctx.past_len, ctx.n_seqs, 1, self.n_heads,
                                      self.n_kv_heads, self.head_dim, self.scale, causal=self.causal, window=window,
                                      k_pool=k_pool, v_pool=v_pool, table=table, table_len=group.table_len)
        elif ctx.is_decode:
            splits = self._splits(ctx)
            kernels.attention_decode(proj, mixed, k_pool, v_pool, table, group.table_len, ctx.ctx_len, ctx.n_seqs,
                                     self.n_heads, self.n_kv_heads, self.head_dim, self.scale, window=window,
                                     n_splits=splits, max_ctx=ctx.ctx_bound,
                                     new_kv_offsets=(self.q_width, self.q_width + self.kv_width) if owns_cache else None)
        elif ctx.fresh and owns_cache:
            # every sequence starts at position 0: keys and values are the step's own projections
            kernels.attention_prefill(proj, mixed, ctx.seq_start, ctx.past_len, ctx.n_seqs, ctx.max_new,
                                           self.n_heads, self.n_kv_heads, self.head_dim, self.scale,
                                           causal=self.causal, window=window,
                                           k_offset=self.q_width, v_offset=self.q_width + self.kv_width)
        else:
            if group.is_ring and ctx.max_new > group.table_len * PAGE_SIZE - self.window + 1:
                # (the engine refuses such a step before the cache changes; this guards direct users of the part)
                raise CacheError("a step that brings this many tokens to sequences that already hold some would "
                                 "overwrite keys of a windowed layer's ring that its first tokens still see")
            kernels.attention_prefill(proj, mixed, ctx.seq_start, ctx.past_len, ctx.n_seqs, ctx.max_new,
                                           self.n_heads, self.n_kv_heads, self.head_dim, self.scale,
                                           causal=self.causal, window=window, k_pool=k_pool, v_pool=v_pool,
                                           table=table, table_len=group.table_len)
        linear(ctx, mixed, self.t_out_weight, self.t_out_bias if self.has_bias else None, residual, m=n,
               residual=residual, w_is_nk=self.nk_out_weight)
