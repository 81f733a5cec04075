"""Random weights from a configuration and a seed, written as a model folder.

Values come from a counter-based generator (SplitMix64 draws, Box-Muller), keyed by
the seed, the tensor's name and the element's index, so the same seed gives the same
file on every machine and no tensor's values depend on another tensor.
The distributions are those of the reference's GPT-2 initialisation policy
(src/models/gpt2.rs:188-222 of NoahIsCool/burn-transformers): the plan gives each tensor
a normal standard deviation, zeros or ones.

`loud=True` is for tests: with standard deviation 0.02 attention is nearly uniform and
a fault in a mask or a cache slot hardly moves the logits, so the loud mode widens every
matrix, gives biases and shifts values and moves the gains away from one.  The
reference's own fixture generator widens `c_fc` for the same reason
(src/models/gpt2/prepare_reference.py:32-35).
"""
from __future__ import annotations

import json
import os
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np
import torch

from ..config.base import ModelConfig
from ..config.registry import architecture_for
from .safetensors_io import write_file
from .spec import MATRIX, VECTOR, WeightPlan

_G = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def _mix(v: np.ndarray) -> np.ndarray:
    v = (v ^ (v >> np.uint64(30))) * _M1
    v = (v ^ (v >> np.uint64(27))) * _M2
    return v ^ (v >> np.uint64(31))


def _name_key(name: str) -> int:
    """FNV-1a, 64 bit."""
    h = 0xCBF29CE484222325
    for byte in name.encode():
        h = ((h ^ byte) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def standard_normal(seed: int, name: str, count: int) -> np.ndarray:
    """`count` float32 draws of N(0, 1) for tensor `name`.  (Pieces of 4 M elements are independent of one another
    and are drawn by several threads: the result does not depend on how many.)"""
    with np.errstate(over="ignore"):
        stream = _mix(np.array([(seed ^ _name_key(name)) & 0xFFFFFFFFFFFFFFFF], dtype=np.uint64) + _G)[0]
    out = np.empty(count, dtype=np.float32)
    chunk = 1 << 22

    def draw(lo: int) -> None:
        hi = min(count, lo + chunk)
        with np.errstate(over="ignore"):
            k = np.arange(lo, hi, dtype=np.uint64)
            a = _mix(stream + _G * (np.uint64(2) * k + np.uint64(1)))
            b = _mix(stream + _G * (np.uint64(2) * k + np.uint64(2)))
        u1 = ((a >> np.uint64(11)).astype(np.float64) + 0.5) / float(1 << 53)
        u2 = ((b >> np.uint64(11)).astype(np.float64)) / float(1 << 53)
        out[lo:hi] = (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)).astype(np.float32)

    starts = range(0, count, chunk)
    workers = min(len(starts), 16, os.cpu_count() or 1)
    if workers <= 1:
        for lo in starts:
            draw(lo)
    else:
        with ThreadPoolExecutor(max_workers=workers) as pool:
            list(pool.map(draw, starts))
    return out


def _device_normal(seed: int, name: str, count: int, device) -> np.ndarray:
    """`count` float32 draws of N(0, 1) from torch's generator on `device`, seeded by the seed and the tensor's name:
    for large models, where the host generator takes minutes.  Other values than `standard_normal` gives."""
    gen = torch.Generator(device=device)
    gen.manual_seed((seed ^ _name_key(name)) & 0x7FFFFFFFFFFFFFFF)
    return torch.randn(count, generator=gen, device=device, dtype=torch.float32).cpu().numpy()


def random_tensors(plan: WeightPlan, seed: int, *, storage: str = "bfloat16", loud: bool = False,
                   device=None) -> dict[str, torch.Tensor]:
    """Host tensors for every tensor a checkpoint of the plan stores (under its stored name and in its stored
    layout).  Matrices are stored in `storage`, vectors in float32.  `device`: draw on this torch device instead of
    with the host generator (faster, other values)."""
    matrix_dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[storage]
    draw = standard_normal if device is None else (lambda s, n, c: _device_normal(s, n, c, device))
    tensors = {}
    for name, spec in plan.stored().items():
        count = int(np.prod(spec.shape)) if spec.shape else 1
        kind = spec.init[0]
        if kind == "normal":
            std = spec.init[1]
            if loud:
                std = max(std * 8.0, 0.15)
            values = draw(seed, name, count) * np.float32(std)
        elif kind == "zeros":
            values = (draw(seed, name, count) * np.float32(0.1)) if loud else np.zeros(count, np.float32)
        elif kind == "ones":
            values = (1.0 + draw(seed, name, count) * np.float32(0.2)) if loud else np.ones(count, np.float32)
        else:
            raise ValueError(f"unknown init {spec.init} for {name}")
        t = torch.from_numpy(np.ascontiguousarray(values, dtype=np.float32)).reshape(spec.shape)
        tensors[name] = t.to(matrix_dtype) if spec.kind == MATRIX else t
    return tensors


def write_random_model(folder, config: ModelConfig | dict, seed: int, *, storage: str = "bfloat16",
                       loud: bool = False, device=None) -> Path:
    """Writes `config.json` and `model.safetensors` into `folder` and returns it.  `device`: see `random_tensors`."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    if isinstance(config, dict):
        arch = architecture_for(config.get("model_type", ""))
        config = arch.config_class.from_dict(config)
    else:
        arch = architecture_for(config.model_type)
    plan = arch.build(config).weights
    data = config.to_dict()
    data["torch_dtype"] = storage
    (folder / "config.json").write_text(json.dumps(data, indent=1) + "\n")
    write_file(folder / "model.safetensors", random_tensors(plan, seed, storage=storage, loud=loud, device=device),
               metadata={"format": "pt", "seed": str(seed), "loud": str(bool(loud))})
    return folder
