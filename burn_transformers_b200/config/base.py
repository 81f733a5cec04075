"""Typed model configurations read from an architecture's own config.json keys.

A configuration class lists its fields once (name, type, default, aliases);
`from_dict` reads exactly those keys, ignores the rest as the reference's serde
structs do (src/models/gpt2.rs:104-107), and `validate` reports the first broken
invariant as `family.field: reason` (src/models/config.rs:70-80).
"""
from __future__ import annotations

import dataclasses
import json
import math
from pathlib import Path
from typing import Any, ClassVar

from ..errors import ConfigError

# Wrappers under which multimodal checkpoints nest the text model's configuration
# (src/models/config.rs:177-229).
_TEXT_WRAPPERS = ("text_config", "language_config", "llm_config")
MAX_CONFIG_BYTES = 16 << 20  # src/models/auto/load.rs:83
MAX_LAYERS = 1 << 18         # src/models/config.rs:908
I32_MAX = (1 << 31) - 1


def read_json_object(path: Path) -> dict:
    path = Path(path)
    if not path.is_file():
        raise ConfigError("config", "config.json", f"{path} does not exist")
    if path.stat().st_size > MAX_CONFIG_BYTES:
        raise ConfigError("config", "config.json", f"larger than {MAX_CONFIG_BYTES} bytes")
    try:
        data = json.loads(path.read_text())      # (json reads Infinity and NaN as they stand)
    except json.JSONDecodeError as error:
        raise ConfigError("config", "config.json", f"not valid JSON: {error}") from None
    if not isinstance(data, dict):
        raise ConfigError("config", "config.json", "must hold a JSON object")
    return data


def detect_model_type(data: dict) -> str:
    """The `model_type` string of a direct or wrapped configuration (src/models/auto.rs:1262-1282)."""
    value = data.get("model_type")
    if value is None:
        for wrapper in _TEXT_WRAPPERS:
            inner = data.get(wrapper)
            if isinstance(inner, dict) and "model_type" in inner:
                value = inner["model_type"]
                break
    if not isinstance(value, str):
        raise ConfigError("config", "model_type", "missing or not a string")
    return value


def field(default, *, aliases=(), doc=""):
    return dataclasses.field(default=default, metadata={"aliases": tuple(aliases), "doc": doc})


@dataclasses.dataclass
class ModelConfig:
    """Base of every architecture's configuration."""

    FAMILY: ClassVar[str] = "model"
    MODEL_TYPES: ClassVar[tuple[str, ...]] = ()

    @classmethod
    def from_dict(cls, data: dict) -> "ModelConfig":
        if not isinstance(data, dict):
            raise ConfigError(cls.FAMILY, "config", "must be a JSON object")
        values: dict[str, Any] = {}
        for f in dataclasses.fields(cls):
            keys = (f.name,) + f.metadata.get("aliases", ())
            present = [k for k in keys if k in data]
            if not present:
                continue
            values[f.name] = cls._coerce(f, data[present[0]])
        config = cls(**values)
        config.validate()
        return config

    @classmethod
    def from_json_file(cls, path) -> "ModelConfig":
        data = read_json_object(Path(path))
        if "model_type" not in data:
            for wrapper in _TEXT_WRAPPERS:
                if isinstance(data.get(wrapper), dict):
                    data = data[wrapper]
                    break
        return cls.from_dict(data)

    @classmethod
    def _coerce(cls, f: dataclasses.Field, value):
        kind = f.type if isinstance(f.type, str) else getattr(f.type, "__name__", str(f.type))
        bad = lambda want: ConfigError(cls.FAMILY, f.name, f"expected {want}, found {value!r}")
        if kind in ("int", "int | None", "Optional[int]"):
            if value is None and "None" in kind:
                return None
            if isinstance(value, bool) or not isinstance(value, int):
                if isinstance(value, float) and value.is_integer():
                    return int(value)
                raise bad("an integer")
            return value
        if kind == "float":
            if isinstance(value, bool) or not isinstance(value, (int, float)):
                raise bad("a number")
            return float(value)
        if kind == "bool":
            if not isinstance(value, bool):
                raise bad("true or false")
            return value
        if kind == "str":
            if not isinstance(value, str):
                raise bad("a string")
            return value
        return value

    def validate(self) -> None:  # pragma: no cover - overridden
        raise NotImplementedError

    def to_dict(self) -> dict:
        return dataclasses.asdict(self)

    # helpers shared by families ------------------------------------------------
    def _fail(self, field_name: str, reason: str):
        raise ConfigError(self.FAMILY, field_name, reason)

    def _check_model_type(self, value: str):
        if value not in self.MODEL_TYPES:
            self._fail("model_type", f"expected one of {list(self.MODEL_TYPES)}, found `{value}`")

    def _check_extents(self, names):
        """First field outside 1..=i32::MAX is named (src/models/gpt2/extents.rs:68-90)."""
        for name in names:
            value = getattr(self, name)
            if value <= 0 or value > I32_MAX:
                self._fail(name, "must be positive and fit the portable integer index range")

    def _check_layer_count(self, name):
        value = getattr(self, name)
        if value == 0:
            self._fail(name, "must be nonzero")
        if value > MAX_LAYERS:
            self._fail(name, f"{value} exceeds the supported maximum of {MAX_LAYERS} layers")

    def _check_positive_finite(self, name):
        value = getattr(self, name)
        if not (math.isfinite(value) and value > 0.0):
            self._fail(name, "must be finite and greater than zero")
