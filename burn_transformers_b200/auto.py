"""Loading a model folder and generating from it, with the reference's names.

    loaded = AutoCausalLm.load_local(folder, AutoLoadOptions(dtype="bfloat16"))
    out = generate_causal(loaded.model, CausalGenerationRequest(prompt=[[464, 1115]], generation=...))

mirrors `AutoCausalLm::load_local(root, &options, &device) -> LoadedModel` and
`generate_causal(model, CausalGenerationRequest{prompt, cache, generation, ..})` of
NoahIsCool/burn-transformers (src/models/auto/load.rs:137-148, src/loaded.rs:212-229,
src/generation/causal.rs:40-62, 100-109).  Prompts are token ids: this library has no tokenizer.
"""
from __future__ import annotations

import dataclasses
from typing import Callable

from .cache.spec import PAGE_SIZE, CacheConfig
from .engine.engine import Engine
from .engine.generate import GenerationToken, generate
from .sampling.config import GenerationConfig
from .sampling.tracker import GeneratedSequence


@dataclasses.dataclass
class AutoLoadOptions:
    dtype: str = "bfloat16"           # "bfloat16" (serving) or "float32" (true 32-bit everywhere)
    device: str = "cuda:0"
    max_tokens: int | None = None     # cache size in tokens; default: one sequence of the longest length
    max_slots: int | None = None
    max_context: int | None = None


@dataclasses.dataclass
class LoadedModel:
    model: Engine
    generation_defaults: GenerationConfig
    source: str
    load_report: list

    @property
    def config(self):
        return self.model.plan.config


class AutoCausalLm:
    @staticmethod
    def load_local(root, options: AutoLoadOptions | None = None) -> LoadedModel:
        options = options or AutoLoadOptions()
        engine = Engine.from_folder(root, options.dtype, max_tokens=options.max_tokens, max_slots=options.max_slots,
                                    max_context=options.max_context, device=options.device)
        return LoadedModel(engine, GenerationConfig.from_model_folder(root), str(root), engine.load_report)


@dataclasses.dataclass
class CausalGenerationRequest:
    prompt: list[list[int]]
    generation: GenerationConfig = dataclasses.field(default_factory=GenerationConfig)
    max_batch: int | None = None
    # the most tokens of a prompt one step brings; None: whole prompts in one step (src/generation/causal.rs:49-59)
    prefill_chunk_size: int | None = None


@dataclasses.dataclass
class CausalGenerationOutput:
    sequences: list[GeneratedSequence]


def generate_causal(model: Engine, request: CausalGenerationRequest) -> CausalGenerationOutput:
    return CausalGenerationOutput(generate(model, request.prompt, request.generation, max_batch=request.max_batch,
                                           prefill_chunk_size=request.prefill_chunk_size))


def generate_causal_streaming(model: Engine, request: CausalGenerationRequest,
                              on_token: Callable[[GenerationToken], None]) -> CausalGenerationOutput:
    return CausalGenerationOutput(generate(model, request.prompt, request.generation, max_batch=request.max_batch,
                                           on_token=on_token, prefill_chunk_size=request.prefill_chunk_size))


def cache_tokens_for(prompt_lengths: list[int], max_new_tokens: int) -> int:
    """Tokens a cache must hold to serve these prompts as one batch."""
    return sum(-(-(n + max_new_tokens - 1) // PAGE_SIZE) * PAGE_SIZE for n in prompt_lengths)
