"""Decode steps as CUDA graphs.

A step in which every sequence brings one token always launches the same kernels with the same
arguments; only the integers they read (tokens, positions, lengths, page tables) change.  Those live
in one device buffer with a fixed layout, so the launches are recorded once per batch size and
replayed: one graph launch per step instead of some seventy kernel launches from Python.

Two recordings exist per batch size: the forward pass alone (`Engine.step` uses it, the host sends the
integers every step), and forward + token selection + advance (`DecodeSession` uses it: the selected
ids become the next step's tokens on the device, so the host only launches and reads results, one
step behind).
"""
from __future__ import annotations

import gc
import weakref

import numpy as np
import torch

from .. import kernels
from ..errors import KernelError
from ..errors import GenerationError
from .step import PinnedStaging, StepContext, Workspace


def _align4(n: int) -> int:
    return (n + 3) & ~3


class DecodeMeta:
    """The integers of a decode step for `n` sequences, in pinned host memory and on the device."""
    SECTIONS = ("tokens", "positions", "token_seq", "seq_start", "past_len", "ctx_len", "slots", "want_rows", "counters")

    def __init__(self, n: int, table_width: int, n_groups: int, device):
        self.n, self.table_width, self.n_groups = n, table_width, n_groups
        sizes = {name: n for name in self.SECTIONS}
        sizes["seq_start"] = n + 1
        self.offsets, total = {}, 0
        for name in self.SECTIONS:
            self.offsets[name] = total
            total += _align4(sizes[name])
        self.table_offsets = []
        for _ in range(n_groups):
            self.table_offsets.append(total)
            total += _align4(n * table_width)
        self.total = total
        self.sizes = sizes
        # two pinned buffers in turn: the host never rewrites integers whose copy to the device has not run yet
        self.staging = PinnedStaging(total)
        self.dev = torch.zeros(total, dtype=torch.int32, device=device)
        ar = np.arange(n + 1, dtype=np.int32)
        for self.host_np in self.staging.arrays:      # the sections that never change, in both buffers
            self._set("token_seq", ar[:n])
            self._set("seq_start", ar)
            self._set("want_rows", ar[:n])
        # results of the selection kernel: ids, then the log-probabilities' bits
        self.out = torch.zeros(2 * n, dtype=torch.int32, device=device)
        self.seeds = torch.zeros(n, dtype=torch.int64, device=device)

    def _set(self, name, values):
        off = self.offsets[name]
        self.host_np[off:off + len(values)] = values

    def view(self, name) -> torch.Tensor:
        off = self.offsets[name]
        return self.dev[off:off + self.sizes[name]]

    def table(self, g) -> torch.Tensor:
        off = self.table_offsets[g]
        return self.dev[off:off + self.n * self.table_width].view(self.n, self.table_width)

    def fill(self, tokens, pasts, slots, tables, counters=None):
        """tables: per group, a list of page lists (one per sequence)."""
        _, self.host_np = self.staging.next_buffer()
        pasts = np.asarray(pasts, dtype=np.int32)
        self._set("tokens", np.asarray(tokens, dtype=np.int32))
        self._set("positions", pasts)
        self._set("past_len", pasts)
        self._set("ctx_len", pasts + 1)
        self._set("slots", np.asarray(slots, dtype=np.int32))
        if counters is not None:
            self._set("counters", np.asarray(counters, dtype=np.int32))
        for g, rows in enumerate(tables):
            off = self.table_offsets[g]
            flat = np.zeros((self.n, self.table_width), dtype=np.int32)
            for i, row in enumerate(rows):
                flat[i, :len(row)] = row
            self.host_np[off:off + self.n * self.table_width] = flat.reshape(-1)

    def upload(self):
        self.staging.copy_to(self.dev, self.total)
        return self.total * 4


class DecodeGraph:
    """The recorded decode step of `n` sequences, with or without token selection."""

    def __init__(self, engine, n: int, selection: dict | None = None):
        # no strong reference back to the engine: a recording must die with its engine at once, by reference
        # count, and never later inside the garbage collector while another recording is being made
        self._engine = weakref.ref(engine)
        self.n, self.selection = n, selection
        cache = engine.cache
        self.meta = DecodeMeta(n, cache.table_width, len(cache.groups), engine.device)
        self.ws = Workspace(engine.device)
        m = self.meta
        self.ctx = StepContext(
            dtype=engine.dtype, cache=cache, ws=self.ws, n_tokens=n, n_seqs=n, n_want=n, max_new=1, is_decode=True,
            fresh=False, ctx_bound=engine.cache_config.max_context, tokens=m.view("tokens"),
            positions=m.view("positions"), token_seq=m.view("token_seq"), seq_start=m.view("seq_start"),
            past_len=m.view("past_len"), ctx_len=m.view("ctx_len"), slots=m.view("slots"),
            want_rows=m.view("want_rows"), tables=[m.table(g) for g in range(len(cache.groups))])
        self.graph = None
        self.program = None        # the fused step, where the model and the batch size allow it
        self.logits = None
        self.launches = 0          # kernels inside one replay

    def _record_program(self):
        """Records the step as the phase program of the fused decode kernel; None if something has no phase."""
        from .program import DecodeProgram, ProgramUnsupported
        engine = self._engine()
        if engine.dtype != torch.bfloat16 or not getattr(engine, "use_fused_step", True):
            return None
        try:
            program = DecodeProgram(engine.device, self.n)
            self.ws.reset()
            self.ctx.program = program
            logits = engine.plan.forward(self.ctx)
            if self.selection is not None:
                program.add_sample(logits, self.meta, self.selection)
            program.finalize()
            self.logits = logits
            return program
        except ProgramUnsupported:
            return None
        finally:
            self.ctx.program = None

    def _settle(self, keep):
        """Makes the workspace one buffer that holds a whole step with room to spare; `keep` (a result that lies in
        it) is copied out first if the buffer has to move."""
        ws = self.ws
        need = ws.offset + (1 << 16)
        if ws._retired or ws.buffer.numel() < need:
            torch.cuda.current_stream().synchronize()
            keep = None if keep is None else keep.clone()
            ws.buffer = torch.empty(max(need, 2 * ws.buffer.numel()), dtype=torch.uint8, device=ws.device)
            ws._typed.clear()
            ws._retired.clear()
        return keep

    def _issue(self):
        """Launches the step's kernels on the current stream (eagerly, or into a recording)."""
        self.ws.reset()
        logits = self._engine().plan.forward(self.ctx)
        if self.selection is not None:
            m, s = self.meta, self.selection
            kernels.sample(logits, self.n, do_sample=s["do_sample"], temperature=s["temperature"], top_k=s["top_k"],
                           top_p=s["top_p"], min_p=s["min_p"], stream_seeds=m.seeds if s["do_sample"] else None,
                           counters=m.view("counters") if s["do_sample"] else None, out_ids=m.out[:self.n],
                           out_logp=m.out[self.n:].view(torch.float32))
            kernels.advance(m.out[:self.n], m.view("tokens"), m.view("positions"), m.view("past_len"),
                            m.view("ctx_len"), m.view("counters"), self.n)
        return logits

    def run(self) -> torch.Tensor:
        """Runs the step on what the device copy of the integers holds.  The first call runs the kernels directly
        and then records them; later calls replay the recording."""
        if self.program is not None:
            try:
                self.program.launch()
                return self.logits
            except KernelError:
                # the launch was refused (a cooperative launch needs every block resident at once, which a GPU that
                # is shared with other work may not grant): this engine goes on with separate kernels
                self.program = None
                self._engine().use_fused_step = False
        if self.graph is not None:
            self.graph.replay()
            return self.logits
        before = kernels.launch_count()
        first = self._issue()
        self.launches = kernels.launch_count() - before
        # a recording must find every piece of scratch at a fixed address: size the workspace for a whole step
        # before recording, and let it grow no more
        first = self._settle(first)
        self.program = self._record_program()
        if self.program is not None and self.ws._retired:
            # the fused step needed more scratch than the separate kernels: make room, then record for good
            first = self._settle(first)
            self.program = self._record_program()
        self.ws.frozen = True
        if self.program is not None:
            self.launches = 2          # the clear of the barrier counter and the step itself
            return first
        first = self._settle(first)
        graph = torch.cuda.CUDAGraph()
        # nothing may free device or pinned memory while the stream records: keep the collector out
        gc.collect()
        was_enabled = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph):
                self.logits = self._issue()
        finally:
            if was_enabled:
                gc.enable()
        self.graph = graph
        return first


class StepGraph:
    """A recorded step of any shape: the kernels of steps that bring the same number of tokens, sequences and
    wanted rows (and the same longest new run) are the same launches with the same arguments, only the integers
    differ.  The engine records a shape when it meets it a second time and replays it afterwards, which takes
    the per-launch cost of the host out of prompts that repeat a shape."""

    def __init__(self, engine):
        from .step import StepBuilder
        self._engine = weakref.ref(engine)
        self.builder = StepBuilder(engine.cache, engine.dtype, engine.device)
        self.graph = None
        self.logits = None
        self.launches = 0

    def run(self, entries):
        engine = self._engine()
        ws = self.builder.ws
        ctx = self.builder.build(entries)          # packs and uploads the step's integers to fixed addresses
        if self.graph is not None:
            self.graph.replay()
            return self.logits
        ws.reset()
        before = kernels.launch_count()
        first = engine.plan.forward(ctx)
        self.launches = kernels.launch_count() - before
        need = ws.offset + (1 << 16)
        if ws._retired or ws.buffer.numel() < need:
            torch.cuda.current_stream().synchronize()
            keep = None if first is None else first.clone()
            ws.buffer = torch.empty(max(need, 2 * ws.buffer.numel()), dtype=torch.uint8, device=ws.device)
            ws._typed.clear()
            ws._retired.clear()
            first = keep
        ws.frozen = True
        graph = torch.cuda.CUDAGraph()
        gc.collect()
        was_enabled = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph):
                ws.reset()
                self.logits = engine.plan.forward(ctx)
        finally:
            if was_enabled:
                gc.enable()
        self.graph = graph
        return first


class DecodeSession:
    """Decodes a fixed set of sequences with the tokens fed forward on the device.

    Each step is one replay of the recorded forward + selection + advance; the host launches step k+1
    before it reads step k's ids, so the device never waits for the host.  A sequence that reaches its
    length limit is known beforehand and leaves before the next launch; one that stops on an
    end-of-sequence token or a stop sequence is found one step late, and that one step's result for it is
    thrown away (its cache row lies in pages the sequence still owns, and its slot is released with it).
    """

    def __init__(self, engine, config, sampler_rows: int):
        self.engine, self.config = engine, config
        self.selection = dict(do_sample=config.samples, temperature=float(config.temperature),
                              top_k=int(config.top_k) if (config.samples and config.top_k and config.top_k < engine.plan.vocab) else 0,
                              top_p=float(config.top_p) if (config.samples and config.top_p is not None) else 1.0,
                              min_p=float(config.min_p) if (config.samples and config.min_p is not None) else 0.0)
        self.host_out = [torch.zeros(2 * sampler_rows, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self.events = [torch.cuda.Event() for _ in range(2)]
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.steps = 0

    @staticmethod
    def usable(engine, config) -> bool:
        return engine.use_graphs and not config.edits_logits and config.counter_mode == "per_sequence"

    def _compose(self, trackers, slots):
        """Uploads the state of the sequences that go on: their last token, length, pages, stream and counter."""
        from ..sampling.random import sequence_stream
        engine, cache = self.engine, self.engine.cache
        graph = engine.decode_graph(len(trackers), self.selection)
        meta = graph.meta
        meta.fill([t.output.token_ids[-1] for t in trackers], [cache.length(slots[t.request]) for t in trackers],
                  [slots[t.request] for t in trackers],
                  [[cache.table_row(g, slots[t.request]) for t in trackers] for g in range(len(cache.groups))],
                  counters=[t.emitted for t in trackers])
        self.h2d_bytes += meta.upload()
        if self.config.samples:
            seeds = np.array([sequence_stream(self.config.seed, t.request) for t in trackers], dtype=np.uint64)
            meta.seeds.copy_(torch.from_numpy(seeds.view(np.int64)), non_blocking=False)
            self.h2d_bytes += 8 * len(trackers)
        return graph

    def run(self, trackers, slots, emit):
        """`trackers`: unfinished sequences, each having emitted at least one token.  `emit(tracker, id, logp)`
        records a token and returns the finish reason or None."""
        engine, cache, cfg = self.engine, self.engine.cache, self.config
        active = list(trackers)
        # all pages a sequence can still need: prompt + max_new_tokens - 1 positions
        cache.reserve([(slots[t.request], len(t.prompt) + cfg.max_new_tokens - 1) for t in active])
        while active:
            n = len(active)
            graph = self._compose(active, slots)
            # steps this composition can run before a sequence reaches its length limit
            budget = min(cfg.max_new_tokens - t.emitted for t in active)
            launched, processed = 0, 0
            stop = False
            while processed < launched or (launched < budget and not stop):
                if launched < budget and not stop and launched - processed < 2:
                    graph.run()
                    buf = launched % 2
                    self.host_out[buf][:2 * n].copy_(graph.meta.out, non_blocking=True)
                    self.events[buf].record()
                    launched += 1
                    self.steps += 1
                    self.d2h_bytes += 8 * n
                    if launched - processed < 2 and launched < budget:
                        continue            # keep one step in flight ahead of the host
                buf = processed % 2
                self.events[buf].synchronize()
                ids = self.host_out[buf][:n].tolist()
                logps = self.host_out[buf][n:2 * n].view(torch.float32).tolist()
                processed += 1
                for t, token, logp in zip(active, ids, logps):
                    if t.finished:
                        continue            # the step after its last one: thrown away
                    cache.commit(slots[t.request], cache.length(slots[t.request]) + 1)
                    if emit(t, token, logp) is not None:
                        stop = True         # the composition changes: drain what is in flight, then recompose
            active = [t for t in active if not t.finished]
