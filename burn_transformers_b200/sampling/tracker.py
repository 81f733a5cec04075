"""Host-side record of what each sequence has emitted, and the decision to stop.

Precedence: an end-of-sequence token, then the longest matching stop sequence (ties: the one
configured first; only once min_new_tokens is reached), then the length limit
(src/generation/bookkeeping.rs:272-296 of the reference).  The end-of-sequence token is emitted
and counted (src/generation/causal.rs:84-85)."""
from __future__ import annotations

import dataclasses


@dataclasses.dataclass(frozen=True)
class FinishReason:
    """kind: "end_of_sequence" (token_id), "stop_sequence" (index, length) or "length"."""
    kind: str
    token_id: int | None = None
    index: int | None = None
    length: int | None = None


def longest_stop_suffix(generated: list[int], stops: list[list[int]]):
    best = None
    for index, stop in enumerate(stops):
        n = len(stop)
        if n and n <= len(generated) and generated[-n:] == list(stop):
            if best is None or n > best[1]:
                best = (index, n)
    return best


def stop_decision(is_eos: bool, token: int, generated: list[int], stops: list[list[int]], min_new_tokens: int,
                  max_new_tokens: int) -> FinishReason | None:
    """None means: go on."""
    if is_eos:
        return FinishReason("end_of_sequence", token_id=token)
    if len(generated) >= min_new_tokens:
        hit = longest_stop_suffix(generated, stops)
        if hit is not None:
            return FinishReason("stop_sequence", index=hit[0], length=hit[1])
    if len(generated) >= max_new_tokens:
        return FinishReason("length")
    return None


@dataclasses.dataclass
class GeneratedSequence:
    prompt_length: int
    token_ids: list[int] = dataclasses.field(default_factory=list)
    log_probabilities: list[float] = dataclasses.field(default_factory=list)
    finish_reason: FinishReason | None = None


class SequenceTracker:
    """One sequence of a generate call: its prompt, what it has emitted, its counts for the penalties."""

    def __init__(self, request: int, prompt: list[int], config):
        self.request = request
        self.prompt = list(prompt)
        self.config = config
        self.output = GeneratedSequence(prompt_length=len(prompt))
        self.counts_generated: dict[int, int] = {}
        self.counts_prompt: dict[int, int] = {}
        if config.repetition_penalty != 1.0 or config.additive_penalty_scope == "prompt_and_generated":
            for t in self.prompt:
                self.counts_prompt[t] = self.counts_prompt.get(t, 0) + 1

    @property
    def finished(self) -> bool:
        return self.output.finish_reason is not None

    @property
    def emitted(self) -> int:
        return len(self.output.token_ids)

    def push(self, token: int, log_probability: float) -> FinishReason | None:
        out = self.output
        out.token_ids.append(token)
        out.log_probabilities.append(log_probability)
        self.counts_generated[token] = self.counts_generated.get(token, 0) + 1
        cfg = self.config
        # an end-of-sequence id cannot be selected before min_new_tokens: its logit is -inf until then
        is_eos = token in cfg.eos_token_ids
        out.finish_reason = stop_decision(is_eos, token, out.token_ids, cfg.stop_sequences, cfg.min_new_tokens,
                                          cfg.max_new_tokens)
        return out.finish_reason

    # ---- edits for the sampler ----------------------------------------------------------
    def banned_tokens(self) -> set[int]:
        """End-of-sequence ids before min_new_tokens, and tokens that would repeat an n-gram."""
        cfg = self.config
        banned: set[int] = set()
        if cfg.eos_token_ids and self.emitted < cfg.min_new_tokens:
            banned.update(cfg.eos_token_ids)
        n = cfg.no_repeat_ngram_size
        if n > 0:
            history = self.prompt + self.output.token_ids
            if len(history) >= n - 1:
                prefix = history[len(history) - (n - 1):] if n > 1 else []
                for i in range(len(history) - n + 1):
                    if history[i:i + n - 1] == prefix:
                        banned.add(history[i + n - 1])
        return banned

    def edits(self) -> dict[int, tuple[float, float, float, float]]:
        """token -> (add, repetition, subtract, ban) in the order bias, repetition penalty, frequency and
        presence penalties, bans (src/generation.rs:605-652, 864-923)."""
        cfg = self.config
        table: dict[int, list[float]] = {}

        def row(token):
            return table.setdefault(int(token), [0.0, 1.0, 0.0, 0.0])

        for token, bias in cfg.logit_bias.items():
            row(token)[0] += float(bias)
        if cfg.repetition_penalty != 1.0:
            for token in set(self.counts_prompt) | set(self.counts_generated):
                row(token)[1] = float(cfg.repetition_penalty)
        if cfg.presence_penalty != 0.0 or cfg.frequency_penalty != 0.0:
            counts = dict(self.counts_generated)
            if cfg.additive_penalty_scope == "prompt_and_generated":
                for token, c in self.counts_prompt.items():
                    counts[token] = counts.get(token, 0) + c
            for token, c in counts.items():
                if c > 0:
                    row(token)[2] += cfg.frequency_penalty * c + cfg.presence_penalty
        for token in self.banned_tokens():
            row(token)[3] = 1.0
        return {t: tuple(v) for t, v in table.items()}
