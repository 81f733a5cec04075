"""The generation loop above the step function.

Requests are served in batches that start together: all prompts of a batch run in one step,
then every unfinished sequence gets one token per step; a sequence that stops leaves the
batch and neither emits nor touches the cache again (src/generation/causal.rs:16-20, 118-211 of
NoahIsCool/burn-transformers).  When a batch has ended its slots are given back and the next
batch starts, until every request is served.

The loop only decides; it asks an engine for logits and a sampler for ids, so its decisions can
be tested with stand-ins for both.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Callable

from ..cache.spec import PAGE_SIZE
from ..errors import GenerationError
from ..sampling.config import GenerationConfig
from ..sampling.tracker import FinishReason, GeneratedSequence, SequenceTracker
from .step import StepEntry


@dataclasses.dataclass
class GenerationToken:
    """One emitted token, as handed to a streaming callback (src/generation/causal.rs:64-77)."""
    sequence: int
    step: int
    token_id: int
    log_probability: float
    finish_reason: FinishReason | None


def pages(tokens: int) -> int:
    return -(-tokens // PAGE_SIZE)


def plan_batches(prompt_lengths: list[int], max_new_tokens: int, *, max_tokens: int, max_slots: int,
                 max_context: int, max_batch: int | None = None) -> list[list[int]]:
    """Cuts the requests, in order, into batches that fit the cache.

    A sequence may grow to prompt + max_new_tokens - 1 cached tokens (the last emitted token is
    never fed back; src/generation/bookkeeping.rs:742-747); a batch fits when the sum of those
    lengths, each rounded up to a whole page, stays within max_tokens and its size within
    max_slots (and max_batch)."""
    limit = min(max_slots, max_batch) if max_batch else max_slots
    if limit <= 0:
        raise GenerationError("max_batch must be greater than zero")
    batches: list[list[int]] = []
    current: list[int] = []
    used = 0
    for index, n in enumerate(prompt_lengths):
        if n <= 0:
            raise GenerationError(f"prompt {index} is empty: every sequence needs at least one token")
        longest = n + max_new_tokens - 1
        if longest > max_context:
            raise GenerationError(f"prompt {index}: {n} prompt tokens + {max_new_tokens} new tokens need "
                                  f"{longest} positions, the cache allows {max_context}")
        need = pages(longest) * PAGE_SIZE
        if need > max_tokens:
            raise GenerationError(f"prompt {index}: needs {need} cached tokens, the cache holds {max_tokens}")
        if current and (used + need > max_tokens or len(current) >= limit):
            batches.append(current)
            current, used = [], 0
        current.append(index)
        used += need
    if current:
        batches.append(current)
    return batches


def _emit(t: SequenceTracker, token: int, logp: float, on_token):
    if not math.isfinite(logp):
        raise GenerationError(f"sequence {t.request}: the selected token {token} has a non-finite "
                              f"log-probability {logp}; generation stops before emitting it")
    reason = t.push(int(token), float(logp))
    if on_token is not None:
        on_token(GenerationToken(t.request, t.emitted - 1, int(token), float(logp), reason))
    return reason


def prefill_prompts(engine, trackers: list[SequenceTracker], slots: dict, chunk: int | None):
    """Runs the batch's prompts and returns the logits at each prompt's last token, one row per tracker.

    Without a chunk size all prompts run in ONE step.  With one, every step brings at most `chunk` tokens of each
    prompt that still has some (src/generation/causal.rs:49-59, 341-396 of the reference: prompts are cut by columns;
    a sequence whose prompt has ended sits out the later portions); only the portion that ends a prompt asks for
    logits, so the rows come from different steps and are gathered here.  Chunked and one-shot prefill give the same
    logits beyond rounding."""
    if chunk is None or chunk >= max(len(t.prompt) for t in trackers):
        return engine.step([StepEntry(slots[t.request], t.prompt, [len(t.prompt) - 1]) for t in trackers])
    gathered = None
    for start in range(0, max(len(t.prompt) for t in trackers), chunk):
        entries, ending = [], []
        for row, t in enumerate(trackers):
            if start >= len(t.prompt):
                continue
            piece = t.prompt[start:start + chunk]
            ends = start + len(piece) == len(t.prompt)
            entries.append(StepEntry(slots[t.request], piece, [len(piece) - 1] if ends else []))
            if ends:
                ending.append(row)
        logits = engine.step(entries)
        if not ending:
            continue
        if hasattr(logits, "new_empty"):
            if gathered is None:
                gathered = logits.new_empty((len(trackers), logits.shape[1]))
            gathered[ending] = logits        # (the step's logits lie in scratch memory the next step reuses)
        else:                                # a stand-in engine's rows (tests of the loop's decisions)
            gathered = gathered or [None] * len(trackers)
            for row, value in zip(ending, logits):
                gathered[row] = value
    return gathered


def run_batch(engine, sampler, trackers: list[SequenceTracker], on_token: Callable | None = None,
              session=None, prefill_chunk_size: int | None = None) -> None:
    """Serves one batch to its end.  `engine` needs new_sequence/step/release; `sampler` needs select.
    With a `session` (engine.graphs.DecodeSession) the one-token steps run from a recorded CUDA graph with
    the selected tokens fed forward on the device."""
    slots = {}
    try:
        for t in trackers:
            slots[t.request] = engine.new_sequence()
        for row, t in enumerate(trackers):
            t.row_in_batch = row
        logits = prefill_prompts(engine, trackers, slots, prefill_chunk_size)
        active = list(trackers)
        batch_rows = len(trackers)
        while active:
            ids, logps = sampler.select(logits, active, batch_rows)
            active = [t for t, token, logp in zip(active, ids, logps) if _emit(t, token, logp, on_token) is None]
            if not active:
                break
            if session is not None:
                session.run(active, slots, lambda t, token, logp: _emit(t, token, logp, on_token))
                break
            logits = engine.step([StepEntry(slots[t.request], [t.output.token_ids[-1]], [0]) for t in active])
        check = getattr(engine, "check_kernels", None)
        if check is not None:
            check()          # (the host has read this batch's last tokens: nothing is in flight)
    finally:
        for slot in slots.values():
            engine.release(slot)


def generate(engine, prompts: list[list[int]], config: GenerationConfig, *, max_batch: int | None = None,
             on_token: Callable | None = None, sampler=None,
             prefill_chunk_size: int | None = None) -> list[GeneratedSequence]:
    """Generates a continuation for every prompt; results come in the order of the prompts.
    `prefill_chunk_size`: the most tokens of a prompt one step brings (None: whole prompts in one step)."""
    vocab = engine.plan.vocab
    config.validate(vocab)
    if not prompts:
        raise GenerationError("generation needs at least one prompt")
    if prefill_chunk_size is not None:
        if prefill_chunk_size <= 0:
            raise GenerationError("prefill_chunk_size must be greater than zero")
        longest_run = getattr(getattr(engine, "cache", None), "max_continued_run", None)
        if longest_run is not None and prefill_chunk_size > longest_run:
            raise GenerationError(f"prefill_chunk_size {prefill_chunk_size} exceeds the {longest_run} tokens a step may "
                                  f"add to a sequence that already holds some (the model has windowed layers)")
    cache = engine.cache_config
    batches = plan_batches([len(p) for p in prompts], config.max_new_tokens, max_tokens=cache.max_tokens,
                           max_slots=cache.max_slots, max_context=cache.max_context, max_batch=max_batch)
    if sampler is None:
        from ..sampling.sampler import DeviceSampler
        sampler = DeviceSampler(config, vocab, engine.device, max(len(b) for b in batches))
    trackers = [SequenceTracker(i, p, config) for i, p in enumerate(prompts)]
    session = None
    if getattr(engine, "use_graphs", False):
        from .graphs import DecodeSession
        if DecodeSession.usable(engine, config):
            session = DecodeSession(engine, config, max(len(b) for b in batches))
    for batch in batches:
        run_batch(engine, sampler, [trackers[i] for i in batch], on_token, session, prefill_chunk_size)
    if session is not None:
        engine.last_session = session
    return [t.output for t in trackers]
