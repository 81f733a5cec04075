"""One step of a batch: the tokens it brings, where they sit, and the scratch memory of the step."""
from __future__ import annotations

import dataclasses

import numpy as np
import torch

from ..errors import KernelError


@dataclasses.dataclass
class StepEntry:
    """A sequence's share of a step: its slot, its next tokens, and the places among these tokens
    (0-based) whose logits are wanted."""
    slot: int
    tokens: list[int]
    want: list[int]


class Workspace:
    """Scratch memory of a step: one device buffer handed out piece by piece and reused every step."""

    def __init__(self, device, initial_bytes: int = 1 << 20):
        self.device = torch.device(device)
        self.buffer = torch.empty(initial_bytes, dtype=torch.uint8, device=self.device)
        self._typed: dict = {}     # flat views of the buffer per element type
        self.offset = 0
        self.frozen = False       # set while a CUDA graph is captured or replayed: addresses must not move
        self._retired: list[torch.Tensor] = []

    def reset(self) -> None:
        self.offset = 0
        self._retired.clear()

    _SIZES = {torch.float32: 4, torch.bfloat16: 2, torch.int32: 4, torch.float16: 2, torch.int64: 8, torch.uint8: 1}

    def take(self, shape, dtype) -> torch.Tensor:
        count = 1
        for s in shape:
            count *= int(s)
        size = self._SIZES.get(dtype) or torch.empty((), dtype=dtype).element_size()
        nbytes = count * size
        start = (self.offset + 255) & ~255
        if start + nbytes > self.buffer.numel():
            if self.frozen:
                raise KernelError("the step's workspace would have to grow while a CUDA graph holds its address")
            # grow: earlier pieces of this step stay valid in the retired buffer
            self._retired.append(self.buffer)
            self.buffer = torch.empty(max(2 * self.buffer.numel(), start + nbytes + (1 << 20)), dtype=torch.uint8,
                                      device=self.device)
            self._typed.clear()
            start = 0
        self.offset = start + nbytes
        flat = self._typed.get(dtype)
        if flat is None or flat.data_ptr() != self.buffer.data_ptr():
            usable = self.buffer.numel() // size * size
            flat = self.buffer[:usable].view(dtype)
            self._typed[dtype] = flat
        first = start // size
        return flat[first:first + count].view(shape)


class StepContext:
    """Everything a part may ask about the step it runs in."""

    def __init__(self, *, dtype, cache, ws, n_tokens, n_seqs, n_want, max_new, is_decode, fresh, ctx_bound,
                 tokens, positions, token_seq, seq_start, past_len, ctx_len, slots, want_rows, tables,
                 host_slots=None, host_seq_start=None, host_past_len=None):
        self.dtype = dtype
        self.cache, self.ws = cache, ws
        self.n_tokens, self.n_seqs, self.n_want, self.max_new = n_tokens, n_seqs, n_want, max_new
        self.is_decode = is_decode      # every sequence brings exactly one token
        self.fresh = fresh              # every sequence starts at position 0
        self.ctx_bound = ctx_bound      # no sequence is longer than this after the step
        # int32 device tensors
        self.tokens, self.positions, self.token_seq = tokens, positions, token_seq
        self.seq_start, self.past_len, self.ctx_len, self.slots = seq_start, past_len, ctx_len, slots
        self.want_rows = want_rows
        self.tables = tables            # per cache group: [n_seqs, table_width] page ids
        self.program = None             # set while a fused decode step is recorded (engine.program.DecodeProgram)
        self.side = None                # a SideWork: a second stream for work nothing later in the step waits for
        # the same facts as Python lists, for parts that plan on the host
        self.host_slots, self.host_seq_start, self.host_past_len = host_slots, host_seq_start, host_past_len


class SideWork:
    """A second stream beside the step's own, for kernels whose results nothing later in the same step reads (filing
    a prompt's keys and values in the pages while attention runs on the step's own projections).

    `fork()` makes the side stream wait for what the step's stream has been given so far; work launched inside
    `with side.stream_context():` then runs beside the step; `join()` makes the step's stream wait for it.  A part
    calls `fork` and the context; the model's forward calls `join` once at the end of the step, before the step's
    scratch memory may be used again.  Inside a stream capture the same calls become a branch of the graph."""

    def __init__(self, device):
        self.stream = torch.cuda.Stream(device=device)
        self.pending = False

    def fork(self):
        event = torch.cuda.Event()
        event.record(torch.cuda.current_stream())
        self.stream.wait_event(event)

    def stream_context(self):
        self.pending = True
        return torch.cuda.stream(self.stream)

    def join(self):
        if self.pending:
            event = torch.cuda.Event()
            event.record(self.stream)
            torch.cuda.current_stream().wait_event(event)
            self.pending = False


def _align4(n: int) -> int:
    return (n + 3) & ~3


class PinnedStaging:
    """Two pinned host buffers of int32, used in turn, each with the event of its last copy to the device.

    A copy from pinned memory is asynchronous: it runs when the stream reaches it, which may be long after the call
    returned (a step whose logits nobody reads is never waited for).  The host must not write the next step's
    integers into a buffer whose copy has not run yet, or the earlier step would run with the later step's
    tokens, positions and page tables.  `next_buffer` therefore waits for the buffer's last copy before handing it
    out; with two buffers the host may run two steps ahead of the device before it waits at all."""

    def __init__(self, count: int, pinned: bool = True):
        self.count = count
        self.pinned = pinned
        self.buffers = [torch.zeros(count, dtype=torch.int32, pin_memory=pinned) for _ in range(2)]
        self.arrays = [b.numpy() for b in self.buffers]
        self.events = [None, None]
        self.turn = 0

    def next_buffer(self):
        """(tensor, numpy view) of the buffer to fill now; waits until its previous copy has run."""
        self.turn ^= 1
        event = self.events[self.turn]
        if event is not None:
            event.synchronize()
        return self.buffers[self.turn], self.arrays[self.turn]

    def copy_to(self, device_tensor: torch.Tensor, count: int) -> None:
        """Queues the copy of the current buffer's first `count` integers and remembers when it has run."""
        device_tensor[:count].copy_(self.buffers[self.turn][:count], non_blocking=True)
        if self.pinned:
            if self.events[self.turn] is None:
                self.events[self.turn] = torch.cuda.Event()
            self.events[self.turn].record()


class StepBuilder:
    """Turns a step's entries into a StepContext: packs the tokens, computes positions from the cache's
    lengths, and sends all integer tables of the step to the device in one copy from pinned memory."""

    def __init__(self, cache, dtype, device):
        self.cache, self.dtype, self.device = cache, dtype, torch.device(device)
        self.ws = Workspace(self.device)
        self._host = None
        self._dev = None
        self.h2d_bytes_last = 0
        self._side = None         # the steps' second stream (made at the first step on a CUDA device)

    def build(self, entries: list[StepEntry]) -> StepContext:
        cache = self.cache
        n_seqs = len(entries)
        pasts = [cache.length(e.slot) for e in entries]
        news = [len(e.tokens) for e in entries]
        seq_start = [0]
        for n in news:
            seq_start.append(seq_start[-1] + n)
        n_tokens = seq_start[-1]
        want_rows = [seq_start[i] + int(w) for i, e in enumerate(entries) for w in e.want]
        ctx_len = [p + n for p, n in zip(pasts, news)]
        slots = [e.slot for e in entries]
        width = cache.table_width
        sizes = [n_tokens, n_tokens, n_tokens, n_seqs + 1, n_seqs, n_seqs, n_seqs, len(want_rows)]
        sizes += [n_seqs * width] * len(cache.groups)
        offsets, total = [], 0
        for size in sizes:
            offsets.append(total)
            total += _align4(max(1, size))
        if self._host is None or self._host.count < total:
            cap = max(total, 4096)
            # (the old buffers stay alive until their copies have run: torch keeps pinned memory of a queued copy)
            self._host = PinnedStaging(cap, pinned=self.device.type == "cuda")
            self._dev = torch.empty(cap, dtype=torch.int32, device=self.device)
        _, h = self._host.next_buffer()
        # the host library fills the buffer (csrc/host/page_book.cpp: positions from the lengths in its books, the
        # page tables from its page lists)
        flat_tokens = np.fromiter((t for e in entries for t in e.tokens), dtype=np.int32, count=n_tokens)
        flat_wants = np.fromiter((int(w) for e in entries for w in e.want), dtype=np.int32, count=len(want_rows))
        counts = np.asarray(news, dtype=np.int32)
        want_counts = np.asarray([len(e.want) for e in entries], dtype=np.int32)
        slot_ids = np.asarray(slots, dtype=np.int32)
        offs = np.asarray(offsets, dtype=np.int64)
        summary = np.zeros(6, dtype=np.int32)
        if cache._lib.bth_book_pack_step(cache._book, n_seqs, slot_ids.ctypes.data, counts.ctypes.data,
                                         flat_tokens.ctypes.data, want_counts.ctypes.data, flat_wants.ctypes.data, width,
                                         offs.ctypes.data, h.ctypes.data, summary.ctypes.data) < 0:
            from ..cache import native
            raise native.error()
        self._host.copy_to(self._dev, total)
        self.h2d_bytes_last = total * 4
        dev = self._dev
        view = lambda i: dev[offsets[i]:offsets[i] + max(1, sizes[i])]
        tables = [view(8 + g).view(n_seqs, width) for g in range(len(cache.groups))]
        tokens = range(n_tokens)
        ctx = StepContext(
            dtype=self.dtype, cache=cache, ws=self.ws, n_tokens=len(tokens), n_seqs=n_seqs, n_want=len(want_rows),
            max_new=max(news), is_decode=all(n == 1 for n in news), fresh=all(p == 0 for p in pasts),
            ctx_bound=max(ctx_len), tokens=view(0), positions=view(1), token_seq=view(2), seq_start=view(3),
            past_len=view(4), ctx_len=view(5), slots=view(6), want_rows=view(7), tables=tables, host_slots=slots,
            host_seq_start=seq_start, host_past_len=pasts)
        if self.device.type == "cuda":
            if self._side is None:
                self._side = SideWork(self.device)
            ctx.side = self._side
        return ctx
