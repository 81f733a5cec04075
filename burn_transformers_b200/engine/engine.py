"""The engine: a model plan with its weights on one GPU, a cache, and the step function.

`step` is the only way tokens reach the model.  A step brings, for each sequence of a batch, its
next tokens (a whole prompt, or one token) and runs exactly those tokens against the cache that
earlier steps left; it returns the 32-bit logits at the wanted places.  Sequences of different
lengths are packed one after another, so there is no padding and nothing to mask out.

The contract follows the reference's prefill/decode pair (src/architecture/traits.rs:110-153,
src/models/shared/rows.rs:1-45 of NoahIsCool/burn-transformers): positions of new tokens continue
the sequence's length, requests are validated before the cache changes, and lengths advance only
when the step has been issued.
"""
from __future__ import annotations

from pathlib import Path

import torch

from .. import kernels
from ..cache import CacheBank, CacheConfig, PAGE_SIZE
from ..config.registry import config_from_folder
from ..errors import CacheError, KernelError, ShapeError
from ..weights.loader import COMPUTE_DTYPES, load_weights
from .model import ModelPlan
from .step import StepBuilder, StepContext, StepEntry


class Engine:
    def __init__(self, plan: ModelPlan, tensors: dict[str, torch.Tensor], dtype: str, cache_config: CacheConfig,
                 device="cuda:0"):
        if dtype not in COMPUTE_DTYPES:
            raise ShapeError(f"dtype must be one of {sorted(COMPUTE_DTYPES)}, found `{dtype}`")
        self.plan = plan
        self.dtype_name = dtype
        self.dtype = COMPUTE_DTYPES[dtype]
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise KernelError(f"the engine runs on a CUDA device only, not on `{device}`")
        kernels.library()  # fail now, loudly, if the kernels cannot be built or loaded
        plan.bind(tensors)
        if cache_config.max_context > plan.max_context:
            raise CacheError(f"cache.max_context {cache_config.max_context} exceeds the model's longest sequence "
                             f"{plan.max_context}")
        self.cache_config = cache_config
        self.cache = CacheBank(plan.cache_needs(), cache_config, self.dtype, self.device)
        self.builder = StepBuilder(self.cache, self.dtype, self.device)
        self.ws = self.builder.ws
        self.steps_run = 0
        # decode steps are replayed from CUDA graphs when every part is made of this library's kernels
        self.use_graphs = plan.graph_safe
        # decode steps as one persistent kernel where the model's parts and the batch size have phases for it
        self.use_fused_step = True
        self.max_graph_batch = 256
        self._graphs: dict = {}
        self._shape_seen: dict = {}        # how often a prefill shape has come by
        self._shape_graphs: dict = {}      # shape -> StepGraph, the most recently used last
        self.max_shape_graphs = 8
        self.h2d_bytes_last = 0

    # ---- construction ------------------------------------------------------------------
    @classmethod
    def from_folder(cls, folder, dtype: str = "bfloat16", *, max_tokens: int | None = None,
                    max_slots: int | None = None, max_context: int | None = None, device="cuda:0") -> "Engine":
        """Reads config.json, picks the architecture by `model_type`, loads model.safetensors strictly."""
        from .. import models  # noqa: F401  (registers the architectures)
        arch, config = config_from_folder(Path(folder))
        plan = arch.build(config)
        tensors, report = load_weights(folder, plan.weights, dtype, torch.device(device))
        max_context = min(max_context or plan.max_context, plan.max_context)
        max_tokens = max_tokens or max_context
        cache_config = CacheConfig(max_tokens=max_tokens, max_slots=max_slots or max(1, -(-max_tokens // PAGE_SIZE)),
                                   max_context=max_context)
        engine = cls(plan, tensors, dtype, cache_config, device)
        engine.load_report = report
        return engine

    # ---- sequences ---------------------------------------------------------------------
    def new_sequence(self) -> int:
        return self.cache.acquire()

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ---- the step ----------------------------------------------------------------------
    def _validate(self, entries: list[StepEntry]) -> None:
        if not entries:
            raise ShapeError("a step needs at least one sequence")
        seen = set()
        vocab = self.plan.vocab
        longest_run = self.cache.max_continued_run
        for e in entries:
            if e.slot in seen:
                raise ShapeError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            past = self.cache.length(e.slot)
            if len(e.tokens) == 0:
                raise ShapeError(f"slot {e.slot}: a step must bring at least one token per sequence")
            if past + len(e.tokens) > self.cache_config.max_context:
                raise CacheError(f"slot {e.slot}: {past} + {len(e.tokens)} tokens exceed the longest sequence of "
                                 f"{self.cache_config.max_context}")
            if longest_run is not None and past > 0 and len(e.tokens) > longest_run:
                raise CacheError(f"slot {e.slot}: a step may add at most {longest_run} tokens to a sequence that already "
                                 f"holds some (the ring of pages of a windowed layer keeps one window only)")
            lo, hi = min(e.tokens), max(e.tokens)
            if lo < 0 or hi >= vocab:
                bad = lo if lo < 0 else hi
                raise ShapeError(f"slot {e.slot}: token id {bad} is outside the vocabulary of {vocab}")
            if e.want and not (0 <= min(e.want) and max(e.want) < len(e.tokens)):
                raise ShapeError(f"slot {e.slot}: wanted place {[w for w in e.want if not 0 <= w < len(e.tokens)][0]} "
                                 f"is outside the {len(e.tokens)} tokens of the step")

    def check_kernels(self) -> None:
        """Raises a KernelError if a kernel of this device reported that a bounded wait of its own ran out."""
        kernels.check_status(self.device)

    def decode_graph(self, n: int, selection: dict | None = None):
        """The recorded decode step for `n` sequences (with token selection when `selection` is given)."""
        from .graphs import DecodeGraph
        key = (n, None if selection is None else tuple(sorted(selection.items())))
        if key not in self._graphs:
            self._graphs[key] = DecodeGraph(self, n, selection)
        return self._graphs[key]

    def _shape_step(self, entries: list[StepEntry]):
        """A step that is not one token per sequence.  A shape met for the second time is recorded as a CUDA graph
        and replayed from then on; the eight most recently used shapes are kept."""
        news = [len(e.tokens) for e in entries]
        shape = (sum(news), len(entries), max(news), sum(len(e.want) for e in entries),
                 all(self.cache.length(e.slot) == 0 for e in entries))
        if self.use_graphs:
            recorded = self._shape_graphs.pop(shape, None)
            seen = self._shape_seen.get(shape, 0)
            self._shape_seen[shape] = seen + 1
            if len(self._shape_seen) > 4096:
                self._shape_seen.clear()
            if recorded is None and seen >= 1:
                from .graphs import StepGraph
                recorded = StepGraph(self)
                while len(self._shape_graphs) >= self.max_shape_graphs:
                    self._shape_graphs.pop(next(iter(self._shape_graphs)))
            if recorded is not None:
                self._shape_graphs[shape] = recorded
                logits = recorded.run(entries)
                self.h2d_bytes_last = recorded.builder.h2d_bytes_last
                return logits
        self.ws.reset()
        ctx = self.builder.build(entries)
        self.h2d_bytes_last = self.builder.h2d_bytes_last
        return self.plan.forward(ctx)

    def _graph_step(self, entries: list[StepEntry]):
        graph = self.decode_graph(len(entries))
        cache = self.cache
        graph.meta.fill([e.tokens[0] for e in entries], [cache.length(e.slot) for e in entries],
                        [e.slot for e in entries],
                        [[cache.table_row(g, e.slot) for e in entries] for g in range(len(cache.groups))])
        self.h2d_bytes_last = graph.meta.upload()
        logits = graph.run()
        wanted = [i for i, e in enumerate(entries) for _ in e.want]
        if wanted == list(range(len(entries))):
            return logits
        if not wanted:
            return None
        return logits[torch.tensor(wanted, device=self.device)]

    def step(self, entries: list[StepEntry]) -> torch.Tensor | None:
        """Runs the entries' tokens as one batch and returns logits [wanted, vocab] (float32, on the device),
        in the order of the entries and of their `want` lists; None when nothing is wanted.

        The returned tensor lies in the step's scratch memory: read it before the next step."""
        self._validate(entries)
        self.cache.reserve([(e.slot, self.cache.length(e.slot) + len(e.tokens)) for e in entries])
        if self.use_graphs and len(entries) <= self.max_graph_batch and all(len(e.tokens) == 1 for e in entries):
            logits = self._graph_step(entries)
        else:
            logits = self._shape_step(entries)
        for e in entries:
            self.cache.commit(e.slot, self.cache.length(e.slot) + len(e.tokens))
        self.steps_run += 1
        return logits
