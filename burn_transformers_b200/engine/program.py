"""The phase program of a fused decode step.

For steps of at most 16 sequences in bfloat16 the whole step can run as one persistent kernel
(csrc/decode_flow.cu) that walks a list of phases.  While a `DecodeProgram` is attached to the step context the
parts do not launch their kernels: `parts.linear.linear`, the attention part and the embedding record a phase
each.  The list is written to the device once per batch size; a step is then one launch.

Inside that kernel the blocks do not meet at barriers: what one phase hands to the next carries a tag that says
which launch wrote it (a bfloat16 value travels as a 32-bit word, a 32-bit value as a 64-bit pair), and a consumer
loads its rows until the tags are the expected ones.  The tensors the parts name (the projections, the attention's
output, the feed-forward's hidden rows, the residual stream) therefore exist twice while a program is recorded: as
the tensor the part holds, which only serves as a name, and as a tagged buffer of the program, which the kernel
uses.  The logits are plain 32-bit numbers in the tensor the readout named.

A part that cannot be expressed as a phase raises `ProgramUnsupported`; the engine then keeps replaying that
batch size from a CUDA graph of the separate kernels.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_uint, c_void_p

import torch

from .. import kernels
from ..cache.spec import PAGE_SIZE

PH_EMBED, PH_LINEAR, PH_ATTENTION, PH_SAMPLE = 0, 1, 2, 3
A_ROWS, A_LAYERNORM, A_RMSNORM = 0, 1, 2
OUT_WORDS, OUT_PAIRS, OUT_PLAIN = 0, 1, 2
MAX_ITEMS = 8          # DF_MAX_ITEMS of csrc/decode_flow.cu
MAX_ROWS = 16
# A tuning knob: a number here replaces the splits an attention phase would choose for itself (tests use it to
# reach the paths of many pages per block and of the merge of several splits).
SPLITS_OVERRIDE = None


# More rows than WIDE_ROWS over layers of WIDE_WEIGHTS weights and more are left to separate kernels (see add_linear).
WIDE_ROWS, WIDE_WEIGHTS = 5, 5_500_000


class ProgramUnsupported(Exception):
    """Something in the step has no phase; the step runs as separate kernels."""


class Phase(ctypes.Structure):
    """Mirror of `bt::FlowPhase` in csrc/decode_flow.cu (same order, same types)."""
    _fields_ = [
        ("type", c_int), ("M", c_int),
        ("a_kind", c_int), ("N", c_int), ("K", c_int), ("act", c_int), ("out_kind", c_int), ("a_src", c_int),
        ("res_src", c_int), ("col_q", c_int),
        ("a", c_void_p), ("rows", c_void_p), ("gamma", c_void_p), ("beta", c_void_p),
        ("eps", c_float), ("col_r", c_int),
        ("w", c_void_p), ("bias", c_void_p), ("out", c_void_p), ("track", c_void_p),
        ("q", c_void_p), ("q_stride", c_longlong), ("k_off", c_int), ("v_off", c_int),
        ("k_pool", c_void_p), ("v_pool", c_void_p), ("table", c_void_p),
        ("table_stride", c_int), ("table_len", c_int),
        ("ctx_len", c_void_p),
        ("n_heads", c_int), ("n_kv_heads", c_int), ("head_dim", c_int), ("n_splits", c_int),
        ("scale_log2", c_float), ("window", c_int),
        ("part", c_void_p), ("attn_out", c_void_p),
        ("tokens", c_void_p), ("positions", c_void_p), ("wte", c_void_p), ("wpe", c_void_p), ("resid", c_void_p),
        ("width", c_int), ("vocab", c_int), ("n_positions", c_int),
        ("do_sample", c_int),
        ("logits", c_void_p),
        ("temperature", c_float), ("top_k", c_int), ("top_p", c_float), ("min_p", c_float),
        ("seeds", c_void_p), ("counters", c_void_p), ("out_ids", c_void_p), ("out_logp", c_void_p),
        ("adv_tokens", c_void_p), ("adv_positions", c_void_p), ("adv_past", c_void_p), ("adv_ctx", c_void_p),
        ("partials", c_void_p), ("n_partials", c_int), ("n_chunks", c_int),
        ("pad3_", ctypes.c_ubyte * 8),                                    # the tensor maps lie on a 64-byte boundary
        ("k_map", ctypes.c_ubyte * 128), ("v_map", ctypes.c_ubyte * 128),
    ]


def _p(t) -> int:
    return 0 if t is None else t.data_ptr()


class DecodeProgram:
    def __init__(self, device, n_rows: int):
        if n_rows > MAX_ROWS:
            raise ProgramUnsupported(f"{n_rows} rows exceed the {MAX_ROWS} a fused step handles")
        lib = kernels.library()
        if lib.bt_decode_flow_phase_bytes() != ctypes.sizeof(Phase):
            raise ProgramUnsupported("the phase layout of the library and of this module differ")
        self.device, self.n_rows = device, n_rows
        self.phases: list[Phase] = []
        self.keep: list = []              # tensors the phases point at
        self.dev = None
        self.plan = None
        self.epoch = 0                    # launches of this program so far: the tag of what a launch writes
        self.counter = torch.zeros(4, dtype=torch.int32, device=device)
        self.n_blocks = torch.cuda.get_device_properties(device).multi_processor_count
        # the tagged buffers, by the address of the tensor a part knows them by
        self.words: dict[int, torch.Tensor] = {}      # bfloat16 values as 32-bit words (value | tag << 16)
        self.pairs: dict[int, torch.Tensor] = {}      # 32-bit values as 64-bit pairs (value, tag)
        self.writer: dict[int, int] = {}              # pairs: index of the phase that wrote them last

    # ---- tagged buffers ----------------------------------------------------------------------------------
    def _new_words(self, t: torch.Tensor) -> torch.Tensor:
        buf = torch.zeros(t.numel(), dtype=torch.int32, device=self.device)
        self.words[t.data_ptr()] = buf
        self.keep += [t, buf]
        return buf

    def _new_pairs(self, t: torch.Tensor) -> torch.Tensor:
        buf = torch.zeros(2 * t.numel(), dtype=torch.int32, device=self.device)
        self.pairs[t.data_ptr()] = buf
        self.keep += [t, buf]
        return buf

    # ---- recording -------------------------------------------------------------------------------------
    def add_embed(self, tokens, positions, wte, wpe, out32):
        if wte.dtype != torch.bfloat16 or wte.shape[1] % 2:
            raise ProgramUnsupported("the fused step is bfloat16 only, with an even width")
        resid = self._new_pairs(out32)
        self.writer[out32.data_ptr()] = len(self.phases)
        ph = Phase(type=PH_EMBED, M=self.n_rows, tokens=_p(tokens), positions=_p(positions), wte=_p(wte), wpe=_p(wpe),
                   resid=_p(resid), width=wte.shape[1], vocab=wte.shape[0],
                   n_positions=0 if wpe is None else wpe.shape[0])
        self._add(ph, tokens, positions, wte, wpe, out32)

    def add_linear(self, a, w, bias, out, *, m, w_is_nk, activation, residual):
        from ..parts.linear import LazyNorm
        if not w_is_nk or w.dtype != torch.bfloat16:
            raise ProgramUnsupported("the fused step needs bfloat16 weights stored [out, in]")
        n, k = w.shape
        if k % 8 or m > MAX_ROWS or w.data_ptr() % 16:
            raise ProgramUnsupported(f"a product of {m} rows and K={k} has no phase")
        if m > WIDE_ROWS and n < 8192 and n * k >= WIDE_WEIGHTS:
            # Layers this large with this many rows are faster as separate kernels: the rows' panel takes the shared
            # memory the weights' ring needs.  Measured a step, fused against separate: width 1280 at 8 rows 2.02
            # against 1.67 ms, at 6 rows 1.62 against 1.58, at 5 rows 1.59 against 1.58, at 4 rows 1.34 against 1.75;
            # width 1600 at 8 rows 3.79 against 3.05, at 5 rows 2.55 against 3.06, at 1 row 1.57 against 2.88; width
            # 1024 at 8 rows 0.97 against 1.02.
            raise ProgramUnsupported(f"a product of {m} rows over {n} x {k} weights is faster outside the fused step")
        index = len(self.phases)
        ph = Phase(type=PH_LINEAR, M=m, N=n, K=k, act=kernels.ACTIVATIONS[activation], w=_p(w), bias=_p(bias),
                   a_src=-1, res_src=-1)
        if isinstance(a, LazyNorm):
            kind = {"layernorm": A_LAYERNORM, "rmsnorm": A_RMSNORM}.get(getattr(a.norm, "fused_kind", None))
            if kind is None:
                raise ProgramUnsupported("this norm cannot be applied inside a product")
            source = a.x32.data_ptr()
            if source not in self.pairs or k > 2304:
                raise ProgramUnsupported("the rows to normalise were not written by a phase of this step")
            ph.a_kind, ph.a, ph.rows, ph.a_src = kind, _p(self.pairs[source]), _p(a.rows), self.writer[source]
            ph.gamma, ph.beta, ph.eps = _p(a.norm.t_weight), _p(a.norm.t_bias if a.norm.has_bias else None), a.norm.eps
            if (ph.gamma or 0) % 16 or (ph.beta or 0) % 16:
                raise ProgramUnsupported("the norm's parameters must lie on 16-byte boundaries")
            self.keep += [a.x32, a.rows]
        else:
            if not isinstance(a, torch.Tensor) or a.dtype != torch.bfloat16 or a.data_ptr() not in self.words:
                raise ProgramUnsupported("the rows of a product must be bfloat16 rows that a phase of this step wrote")
            ph.a_kind, ph.a = A_ROWS, _p(self.words[a.data_ptr()])
            self.keep.append(a)
        if residual is not None:
            target = out.data_ptr()
            if residual.data_ptr() != target or out.dtype != torch.float32 or target not in self.pairs:
                raise ProgramUnsupported("a residual must be the 32-bit stream the product adds to, written by this step")
            ph.out_kind, ph.out, ph.res_src = OUT_PAIRS, _p(self.pairs[target]), self.writer[target]
            self.writer[target] = index
        elif out.dtype == torch.bfloat16:
            ph.out_kind, ph.out = OUT_WORDS, _p(self._new_words(out))
        else:
            ph.out_kind, ph.out = OUT_PLAIN, _p(out)          # the logits: plain numbers, read after the step (or its barrier)
        self._add(ph, w, bias, residual, out)

    def add_attention(self, ctx, proj, k_pool, v_pool, table, table_len, *, n_heads, n_kv_heads, head_dim, scale, window,
                      new_kv_offsets):
        if proj.dtype != torch.bfloat16 or head_dim % 16 or head_dim > 128 or proj.shape[1] % 4:
            raise ProgramUnsupported("attention of this shape has no phase")
        if proj.data_ptr() not in self.words:
            raise ProgramUnsupported("the projections were not written by a phase of this step")
        if new_kv_offsets is None:
            # (the pages would have to hold this step's token already, filed by another phase of the same launch,
            # while the page producer runs ahead of the phases)
            raise ProgramUnsupported("a layer that reads another layer's cache has no phase in the fused step")
        if any(p.type == PH_ATTENTION and p.head_dim != head_dim for p in self.phases):
            raise ProgramUnsupported("the fused step needs one head size in all its attention phases")
        span = ctx.ctx_bound if not window else min(ctx.ctx_bound, window)
        pages = max(1, -(-span // PAGE_SIZE)) + (1 if window else 0)
        units = ctx.n_seqs * n_heads
        # The splits that leave the busiest block the fewest pages (a block takes every n_blocks-th item), among those
        # that give a block at most two items if there are any: an item costs a block a hand-over between its warps
        # and, when it is small, a wait for pages that its ring of slots could not hold ahead (measured: 9 splits
        # of one page each, 8 items a block, took 23.6 us where one item of 9 pages takes 6).
        splits, best = 1, None
        for s in range(1, min(pages, 16) + 1):
            per_block = -(-units * s // self.n_blocks)
            if per_block > MAX_ITEMS:
                break
            load = (per_block > 2, per_block * -(-pages // s))
            if best is None or load < best:
                splits, best = s, load
        if SPLITS_OVERRIDE is not None and -(-units * SPLITS_OVERRIDE // self.n_blocks) <= MAX_ITEMS:
            splits, best = max(1, min(int(SPLITS_OVERRIDE), pages)), (False, 0)
        if best is None:
            raise ProgramUnsupported(f"{units} attention units are too many for the fused step")
        mixed = ctx.ws.take((ctx.n_seqs, n_heads * head_dim), torch.bfloat16)       # the name of the phase's result
        out_words = self._new_words(mixed)
        part = None
        if splits > 1:
            part = torch.zeros(2 * units * splits * (head_dim + 2), dtype=torch.int32, device=self.device)
        ph = Phase(type=PH_ATTENTION, M=ctx.n_seqs, n_splits=splits, n_heads=n_heads, head_dim=head_dim,
                   q=_p(self.words[proj.data_ptr()]), q_stride=proj.shape[1], k_off=new_kv_offsets[0],
                   v_off=new_kv_offsets[1], k_pool=_p(k_pool), v_pool=_p(v_pool), table=_p(table),
                   table_stride=table.shape[1], table_len=table_len, ctx_len=_p(ctx.ctx_len), n_kv_heads=n_kv_heads,
                   scale_log2=scale * 1.4426950408889634, window=window or 0, part=_p(part), attn_out=_p(out_words))
        # the layer's pools as [pages * kv_heads * 64 rows][head_dim]: a page of one head is a box of 64 rows
        lib = kernels.library()
        rows = k_pool.numel() // head_dim
        for pool, field in ((k_pool, "k_map"), (v_pool, "v_map")):
            buf = (ctypes.c_ubyte * 128)()
            kernels._check(lib.bt_tensor_map_2d_bf16(buf, c_void_p(pool.data_ptr()), ctypes.c_ulonglong(rows),
                                                     ctypes.c_ulonglong(head_dim), ctypes.c_ulonglong(head_dim),
                                                     ctypes.c_uint(PAGE_SIZE)))
            setattr(ph, field, buf)
        self._add(ph, proj, k_pool, v_pool, table, part, mixed)
        return mixed

    def add_sample(self, logits, meta, selection):
        ph = Phase(type=PH_SAMPLE, M=self.n_rows, logits=_p(logits), vocab=logits.shape[1],
                   do_sample=1 if selection["do_sample"] else 0, temperature=selection["temperature"],
                   top_k=selection["top_k"], top_p=selection["top_p"], min_p=selection["min_p"],
                   seeds=_p(meta.seeds), counters=_p(meta.view("counters")), out_ids=_p(meta.out),
                   out_logp=meta.out.data_ptr() + 4 * self.n_rows, adv_tokens=_p(meta.view("tokens")),
                   adv_positions=_p(meta.view("positions")), adv_past=_p(meta.view("past_len")),
                   adv_ctx=_p(meta.view("ctx_len")))
        if not selection["do_sample"]:
            # greedy: the readout keeps every block's (max, sum, argmax) of each row; the selection merges them
            # instead of reading the logits again
            readout = next((p for p in reversed(self.phases) if p.type == PH_LINEAR and p.out == logits.data_ptr()), None)
            if readout is not None and readout.out_kind == OUT_PLAIN:
                partials = torch.empty(self.n_rows * self.n_blocks * 4, dtype=torch.float32, device=self.device)
                readout.track = ph.partials = partials.data_ptr()
                ph.n_partials = self.n_blocks
                self.keep.append(partials)
        self._add(ph, logits)

    def _add(self, ph, *tensors):
        self.phases.append(ph)
        self.keep += [t for t in tensors if t is not None]

    # ---- running ---------------------------------------------------------------------------------------
    def finalize(self):
        array = (Phase * len(self.phases))(*self.phases)
        plan = (c_longlong * 8)()
        # (the plan also writes into the phases what the kernel would otherwise divide out: upload after it)
        if kernels.library().bt_decode_flow_plan(ctypes.cast(array, c_void_p), c_int(len(self.phases)),
                                                 c_int(self.n_rows), plan) != 0:
            raise ProgramUnsupported(kernels.library().bt_last_error().decode(errors="replace"))
        host = torch.frombuffer(bytearray(bytes(array)), dtype=torch.uint8)
        self.dev = host.to(self.device)
        self.plan = plan
        self.smem = int(plan[5])

    def launch(self, trace=None):
        """One step.  `trace`: optional int64 tensor of 8 * len(phases) slots for block 0's timeline of each phase."""
        self.epoch = self.epoch % ((1 << 22) - 1) + 1
        kernels._check(kernels.library().bt_decode_flow(
            c_void_p(self.dev.data_ptr()), c_int(len(self.phases)), c_uint(self.epoch), c_int(self.n_rows), self.plan,
            c_void_p(self.counter.data_ptr()), c_void_p(kernels.kernel_status(self.device).data_ptr()),
            c_void_p(0 if trace is None else trace.data_ptr()), kernels._stream()))
