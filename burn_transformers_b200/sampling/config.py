"""Generation controls, with the reference's names, defaults and checks
(src/generation.rs:191-276 and 288-405 of NoahIsCool/burn-transformers)."""
from __future__ import annotations

import dataclasses
import json
import math
import struct
from pathlib import Path

from ..errors import GenerationError

STRATEGIES = ("greedy", "sample")
PENALTY_SCOPES = ("generated", "prompt_and_generated")
COUNTER_MODES = ("per_sequence", "reference")
_F32_SMALLEST_NORMAL = 1.1754943508222875e-38


def _round_f32(value: float) -> float:
    try:
        return struct.unpack("<f", struct.pack("<f", value))[0]
    except OverflowError:
        return math.inf if value > 0 else -math.inf


def _check_divisor(field: str, value: float) -> None:
    if not (math.isfinite(value) and value > 0.0):
        raise GenerationError(f"{field} must be finite and greater than zero")
    rounded = _round_f32(value)
    if not (math.isfinite(rounded) and rounded >= _F32_SMALLEST_NORMAL):
        raise GenerationError(f"{field} {value!r} rounds to {rounded!r} in F32; it must round to a normal positive "
                              f"F32 value")


def _check_finite(field: str, value: float) -> None:
    if not math.isfinite(value) or not math.isfinite(_round_f32(value)):
        raise GenerationError(f"{field} must be finite, found {value!r}")


@dataclasses.dataclass
class GenerationConfig:
    max_new_tokens: int = 256
    min_new_tokens: int = 0
    strategy: str = "greedy"
    temperature: float = 1.0
    top_k: int | None = None
    top_p: float | None = None
    min_p: float | None = None
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    additive_penalty_scope: str = "generated"
    no_repeat_ngram_size: int = 0
    logit_bias: dict[int, float] = dataclasses.field(default_factory=dict)
    seed: int = 0
    eos_token_ids: list[int] = dataclasses.field(default_factory=list)
    pad_token_id: int | None = None
    stop_sequences: list[list[int]] = dataclasses.field(default_factory=list)
    # How uniforms are numbered.  "per_sequence": draw k of request r is splitmix64(splitmix64(seed, r), k), so a
    # request samples the same tokens alone or in any batch.  "reference": the reference's numbering, one block of
    # `batch` counters per step, row b using start + b (src/generation.rs:667-699).
    counter_mode: str = "per_sequence"

    @property
    def samples(self) -> bool:
        return self.strategy == "sample"

    def validate(self, vocabulary_size: int) -> None:
        if vocabulary_size <= 0:
            raise GenerationError("vocabulary_size must be greater than zero")
        if self.max_new_tokens <= 0:
            raise GenerationError("max_new_tokens must be greater than zero")
        if self.min_new_tokens > self.max_new_tokens:
            raise GenerationError(f"min_new_tokens {self.min_new_tokens} exceeds max_new_tokens {self.max_new_tokens}")
        if self.strategy not in STRATEGIES:
            raise GenerationError(f"strategy must be one of {list(STRATEGIES)}, found {self.strategy!r}")
        if self.counter_mode not in COUNTER_MODES:
            raise GenerationError(f"counter_mode must be one of {list(COUNTER_MODES)}, found {self.counter_mode!r}")
        _check_divisor("temperature", self.temperature)
        if self.top_k is not None and not (1 <= self.top_k <= vocabulary_size):
            raise GenerationError(f"top_k must be in 1..={vocabulary_size}, found {self.top_k}")
        if self.top_p is not None and not (math.isfinite(self.top_p) and 0.0 < self.top_p <= 1.0):
            raise GenerationError(f"top_p must be finite and in (0, 1], found {self.top_p}")
        if self.min_p is not None and not (0.0 <= self.min_p <= 1.0):
            raise GenerationError(f"min_p must be in [0, 1], found {self.min_p}")
        _check_divisor("repetition_penalty", self.repetition_penalty)
        _check_finite("presence_penalty", self.presence_penalty)
        _check_finite("frequency_penalty", self.frequency_penalty)
        if self.additive_penalty_scope not in PENALTY_SCOPES:
            raise GenerationError(f"additive_penalty_scope must be one of {list(PENALTY_SCOPES)}")
        if self.no_repeat_ngram_size < 0:
            raise GenerationError("no_repeat_ngram_size must not be negative")
        if not (0 <= self.seed < 1 << 64):
            raise GenerationError("seed must fit 64 unsigned bits")
        special = list(self.eos_token_ids) + ([self.pad_token_id] if self.pad_token_id is not None else [])
        for stop in self.stop_sequences:
            special.extend(stop)
        for token in special:
            if not (0 <= token < vocabulary_size):
                raise GenerationError(f"special token {token} is outside vocabulary size {vocabulary_size}")
        if any(len(stop) == 0 for stop in self.stop_sequences):
            raise GenerationError("stop sequences must not be empty")
        for token, bias in self.logit_bias.items():
            if not (0 <= int(token) < vocabulary_size):
                raise GenerationError(f"logit_bias token {token} is outside vocabulary size {vocabulary_size}")
            _check_finite(f"logit_bias for token {token}", bias)

    @property
    def edits_logits(self) -> bool:
        """Whether any control needs per-token edits before selection."""
        return bool(self.logit_bias) or self.repetition_penalty != 1.0 or self.presence_penalty != 0.0 \
            or self.frequency_penalty != 0.0 or self.no_repeat_ngram_size > 0 \
            or (self.min_new_tokens > 0 and bool(self.eos_token_ids))

    @classmethod
    def from_model_folder(cls, folder) -> "GenerationConfig":
        """Defaults of a checkpoint's generation_config.json, where it has one; else the library defaults."""
        path = Path(folder) / "generation_config.json"
        config = cls()
        if not path.is_file():
            return config
        try:
            data = json.loads(path.read_text())
        except json.JSONDecodeError as error:
            raise GenerationError(f"{path}: not valid JSON: {error}") from None
        if data.get("do_sample") is True:
            config.strategy = "sample"
        for key in ("temperature", "top_k", "top_p", "min_p", "repetition_penalty", "no_repeat_ngram_size",
                    "max_new_tokens", "min_new_tokens"):
            if data.get(key) is not None:
                setattr(config, key, data[key])
        eos = data.get("eos_token_id")
        if isinstance(eos, int):
            config.eos_token_ids = [eos]
        elif isinstance(eos, list):
            config.eos_token_ids = [int(t) for t in eos]
        if isinstance(data.get("pad_token_id"), int):
            config.pad_token_id = data["pad_token_id"]
        return config
