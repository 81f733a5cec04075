"""The phase program of a fused decode step.

For steps of at most 16 sequences in bfloat16 the whole step can run as one persistent kernel
(csrc/decode_step.cu) that walks a list of phases.  While a `DecodeProgram` is attached to the step context the
parts do not launch their kernels: `parts.linear.linear`, the attention part and the embedding record a phase
each.  The list is written to the device once per batch size; a step is then one launch.

A part that cannot be expressed as a phase raises `ProgramUnsupported`; the engine then keeps replaying that
batch size from a CUDA graph of the separate kernels.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .. import kernels
from ..cache.spec import PAGE_SIZE

PH_EMBED, PH_LINEAR, PH_ATTENTION, PH_SAMPLE = 0, 1, 2, 3
MAX_ITEMS = 8          # DS_MAX_ITEMS of csrc/decode_step.cu
# A tuning knob: a number here replaces the splits an attention phase would choose for itself (tests use it to
# reach the paths of many pages per block).
SPLITS_OVERRIDE = None
A_ROWS, A_LAYERNORM, A_MERGE = 0, 1, 2
MAX_ROWS = 16


class ProgramUnsupported(Exception):
    """Something in the step has no phase; the step runs as separate kernels."""


class Phase(ctypes.Structure):
    """Mirror of `bt::Phase` in csrc/decode_step.cu (same order, same types)."""
    _fields_ = [
        ("type", c_int),
        ("a_kind", c_int), ("M", c_int), ("N", c_int), ("K", c_int), ("act", c_int), ("out_is_f32", c_int),
        ("a", c_void_p), ("x32", c_void_p), ("rows", c_void_p), ("gamma", c_void_p), ("beta", c_void_p),
        ("eps", c_float),
        ("part", c_void_p),
        ("n_splits", c_int), ("n_heads", c_int), ("head_dim", c_int),
        ("w", c_void_p), ("bias", c_void_p), ("residual", c_void_p), ("out", c_void_p), ("track", c_void_p),
        ("q", c_void_p), ("q_stride", c_longlong), ("new_k", c_void_p), ("new_v", c_void_p),
        ("k_pool", c_void_p), ("v_pool", c_void_p), ("table", c_void_p),
        ("table_stride", c_int), ("table_len", c_int),
        ("ctx_len", c_void_p),
        ("n_kv_heads", c_int), ("scale_log2", c_float), ("window", c_int),
        ("part_out", c_void_p),
        ("tokens", c_void_p), ("positions", c_void_p), ("wte", c_void_p), ("wpe", c_void_p), ("resid_out", c_void_p),
        ("width", c_int), ("vocab", c_int), ("n_positions", c_int),
        ("logits", c_void_p),
        ("do_sample", c_int), ("temperature", c_float), ("top_k", c_int), ("top_p", c_float), ("min_p", c_float),
        ("seeds", c_void_p), ("counters", c_void_p), ("out_ids", c_void_p), ("out_logp", c_void_p),
        ("adv_tokens", c_void_p), ("adv_positions", c_void_p), ("adv_past", c_void_p), ("adv_ctx", c_void_p),
        ("partials", c_void_p), ("n_partials", c_int), ("pad0_", c_int), ("pad1_", c_longlong),
        ("pad2_", ctypes.c_ubyte * 32),                                   # the tensor maps lie on a 64-byte boundary
        ("k_map", ctypes.c_ubyte * 128), ("v_map", ctypes.c_ubyte * 128),
    ]


class AttentionPartials:
    """What an attention phase leaves: per (sequence, head, split) the weighted values, the maximum and the sum.
    The next matrix product merges them while it builds its rows."""

    def __init__(self, buffer, n_splits, n_heads, head_dim):
        self.buffer, self.n_splits, self.n_heads, self.head_dim = buffer, n_splits, n_heads, head_dim
        self.dtype = torch.bfloat16


def _p(t) -> int:
    return 0 if t is None else t.data_ptr()


class DecodeProgram:
    def __init__(self, device, n_rows: int):
        if n_rows > MAX_ROWS:
            raise ProgramUnsupported(f"{n_rows} rows exceed the {MAX_ROWS} a fused step handles")
        lib = kernels.library()
        if lib.bt_decode_step_phase_bytes() != ctypes.sizeof(Phase):
            raise ProgramUnsupported("the phase layout of the library and of this module differ")
        self.device, self.n_rows = device, n_rows
        self.phases: list[Phase] = []
        self.keep: list = []              # tensors the phases point at
        self.dev = None
        self.smem = 0
        self.counter = torch.zeros(4, dtype=torch.int32, device=device)
        self.n_blocks = torch.cuda.get_device_properties(device).multi_processor_count

    # ---- recording -------------------------------------------------------------------------------------
    def add_embed(self, tokens, positions, wte, wpe, out32):
        if wte.dtype != torch.bfloat16:
            raise ProgramUnsupported("the fused step is bfloat16 only")
        ph = Phase(type=PH_EMBED, M=self.n_rows, tokens=_p(tokens), positions=_p(positions), wte=_p(wte), wpe=_p(wpe),
                   resid_out=_p(out32), width=wte.shape[1], vocab=wte.shape[0],
                   n_positions=0 if wpe is None else wpe.shape[0])
        self._add(ph, tokens, positions, wte, wpe, out32)

    def add_linear(self, a, w, bias, out, *, m, w_is_nk, activation, residual):
        from ..parts.linear import LazyNorm
        if not w_is_nk or w.dtype != torch.bfloat16:
            raise ProgramUnsupported("the fused step needs bfloat16 weights stored [out, in]")
        n, k = w.shape
        if k % 8 or m > MAX_ROWS:
            raise ProgramUnsupported(f"a product of {m} rows and K={k} has no phase")
        ph = Phase(type=PH_LINEAR, M=m, N=n, K=k, act=kernels.ACTIVATIONS[activation],
                   out_is_f32=1 if out.dtype == torch.float32 else 0, w=_p(w), bias=_p(bias), residual=_p(residual),
                   out=_p(out))
        if isinstance(a, LazyNorm):
            if not getattr(a.norm, "fusable", False):
                raise ProgramUnsupported("this norm cannot be applied inside a product")
            ph.a_kind, ph.x32, ph.rows = A_LAYERNORM, _p(a.x32), _p(a.rows)
            ph.gamma, ph.beta, ph.eps = _p(a.norm.t_weight), _p(a.norm.t_bias if a.norm.has_bias else None), a.norm.eps
            if (ph.x32 or 0) % 16 or (ph.gamma or 0) % 16 or (ph.beta or 0) % 16:
                raise ProgramUnsupported("the norm's rows and parameters must lie on 16-byte boundaries")
            self.keep += [a.x32, a.rows]
        elif isinstance(a, AttentionPartials):
            if a.n_heads * a.head_dim != k or a.head_dim % 8:
                raise ProgramUnsupported("attention partials do not match the projection")
            ph.a_kind, ph.part = A_MERGE, _p(a.buffer)
            ph.n_splits, ph.n_heads, ph.head_dim = a.n_splits, a.n_heads, a.head_dim
            self.keep.append(a.buffer)
        else:
            if a.dtype != torch.bfloat16:
                raise ProgramUnsupported("the fused step is bfloat16 only")
            ph.a_kind, ph.a = A_ROWS, _p(a)
            if a.data_ptr() % 16:
                raise ProgramUnsupported("the rows must lie on a 16-byte boundary")
            self.keep.append(a)
        self._add(ph, w, bias, residual, out)

    def add_attention(self, ctx, proj, k_pool, v_pool, table, table_len, *, n_heads, n_kv_heads, head_dim, scale, window,
                      new_kv_offsets):
        if proj.dtype != torch.bfloat16 or head_dim % 16 or head_dim > 128:
            raise ProgramUnsupported("attention of this shape has no phase")
        if any(p.type == PH_ATTENTION and p.head_dim != head_dim for p in self.phases):
            # (pages are numbered through the launch, and a number's slot depends on how many slots a head size gives)
            raise ProgramUnsupported("the fused step needs one head size in all its attention phases")
        span = ctx.ctx_bound if not window else min(ctx.ctx_bound, window)
        pages = max(1, -(-span // PAGE_SIZE)) + (1 if window else 0)
        units = ctx.n_seqs * n_heads
        # the splits that leave the busiest block the fewest pages (a block takes every n_blocks-th item)
        splits, best = 1, None
        for s in range(1, min(pages, 16) + 1):
            per_block = -(-units * s // self.n_blocks)
            if per_block > MAX_ITEMS:
                break
            load = per_block * -(-pages // s)
            if best is None or load < best:
                splits, best = s, load
        if SPLITS_OVERRIDE is not None and -(-units * SPLITS_OVERRIDE // self.n_blocks) <= MAX_ITEMS:
            splits, best = max(1, min(int(SPLITS_OVERRIDE), pages)), 0
        if best is None:
            raise ProgramUnsupported(f"{units} attention units are too many for the fused step")
        part = ctx.ws.take((units * splits * (head_dim + 4),), torch.float32)
        es = proj.element_size()
        ph = Phase(type=PH_ATTENTION, M=ctx.n_seqs, n_splits=splits, n_heads=n_heads, head_dim=head_dim,
                   q=_p(proj), q_stride=proj.shape[1],
                   new_k=(proj.data_ptr() + new_kv_offsets[0] * es) if new_kv_offsets else 0,
                   new_v=(proj.data_ptr() + new_kv_offsets[1] * es) if new_kv_offsets else 0,
                   k_pool=_p(k_pool), v_pool=_p(v_pool), table=_p(table), table_stride=table.shape[1],
                   table_len=table_len, ctx_len=_p(ctx.ctx_len), n_kv_heads=n_kv_heads,
                   scale_log2=scale * 1.4426950408889634, window=window or 0, part_out=_p(part))
        # the layer's pools as [pages * kv_heads * 64 rows][head_dim]: a page of one head is a box of 64 rows
        lib = kernels.library()
        rows = k_pool.numel() // head_dim
        for pool, field in ((k_pool, "k_map"), (v_pool, "v_map")):
            buf = (ctypes.c_ubyte * 128)()
            kernels._check(lib.bt_tensor_map_2d_bf16(buf, c_void_p(pool.data_ptr()), ctypes.c_ulonglong(rows),
                                                     ctypes.c_ulonglong(head_dim), ctypes.c_ulonglong(head_dim),
                                                     ctypes.c_uint(PAGE_SIZE)))
            setattr(ph, field, buf)
        self._add(ph, proj, k_pool, v_pool, table, part)
        return AttentionPartials(part, splits, n_heads, head_dim)

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
            if readout is not None and readout.out_is_f32:
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
        raw = bytes(array)
        host = torch.frombuffer(bytearray(raw), dtype=torch.uint8)
        self.dev = host.to(self.device)
        lib = kernels.library()
        lib.bt_decode_step_smem_bytes.restype = c_longlong
        self.smem = int(lib.bt_decode_step_smem_bytes(ctypes.cast(array, c_void_p), c_int(len(self.phases))))
        self.build = int(lib.bt_decode_step_build(ctypes.cast(array, c_void_p), c_int(len(self.phases))))
        if self.smem > 200 * 1024:
            raise ProgramUnsupported(f"the step needs {self.smem} bytes of shared memory")

    def launch(self, trace=None):
        """One step.  `trace`: optional int64 tensor of 8 * len(phases) slots for block 0's timeline of each phase."""
        kernels._check(kernels.library().bt_decode_step(
            c_void_p(self.dev.data_ptr()), c_int(len(self.phases)), c_int(self.build), c_longlong(self.smem),
            c_void_p(self.counter.data_ptr()), c_void_p(kernels.kernel_status(self.device).data_ptr()),
            c_void_p(0 if trace is None else trace.data_ptr()), kernels._stream()))
