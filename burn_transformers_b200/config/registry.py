"""One registry from an architecture's `model_type` to its configuration class and builder.

The reference keeps such a list in a macro (src/models/auto.rs:299-340, 702-769) and
answers an unknown type with the supported values (src/models/auto.rs:772-777).
An architecture registers itself once; nothing else in the library names a model.
"""
from __future__ import annotations

import dataclasses
from pathlib import Path
from typing import Callable

from ..errors import UnsupportedArchitecture
from .base import ModelConfig, detect_model_type, read_json_object, _TEXT_WRAPPERS


@dataclasses.dataclass(frozen=True)
class Architecture:
    """What the library needs to know about one model family."""
    name: str
    model_types: tuple[str, ...]
    config_class: type
    # build(config) -> engine.model.ModelPlan: the parts, their order and the tensor names
    build: Callable


_REGISTRY: dict[str, Architecture] = {}


def register_architecture(arch: Architecture, *, replace: bool = False) -> Architecture:
    for model_type in arch.model_types:
        if model_type in _REGISTRY and not replace:
            raise ValueError(f"model_type `{model_type}` is already registered")
        _REGISTRY[model_type] = arch
    return arch


def unregister_architecture(model_type: str) -> None:
    _REGISTRY.pop(model_type, None)


def supported_model_types() -> list[str]:
    return sorted(_REGISTRY)


def architecture_for(model_type: str) -> Architecture:
    try:
        return _REGISTRY[model_type]
    except KeyError:
        raise UnsupportedArchitecture(
            f"causal model_type `{model_type}` is not executable; supported values: "
            + ", ".join(supported_model_types())
        ) from None


def config_from_folder(folder) -> tuple[Architecture, ModelConfig]:
    """Reads `folder/config.json`, picks the architecture by `model_type`, returns its typed config."""
    data = read_json_object(Path(folder) / "config.json")
    arch = architecture_for(detect_model_type(data))
    if "model_type" not in data:
        for wrapper in _TEXT_WRAPPERS:
            if isinstance(data.get(wrapper), dict):
                data = data[wrapper]
                break
    return arch, arch.config_class.from_dict(data)
