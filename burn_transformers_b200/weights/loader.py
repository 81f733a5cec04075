"""Strict loading of a model folder's weights by tensor name.

Every name the model expects must be present with the expected shape and a float
dtype, and nothing else may be present, except the names the plan lists as
ignored or tied.  Everything that is wrong is collected and reported in one
error before any tensor is read (src/models/gpt2/checkpoint.rs:223-238, 330-363
of the reference: plan first, then execute).
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..errors import CheckpointError
from . import safetensors_io as st
from .spec import MATRIX, TABLE, VECTOR, Stored, WeightPlan, resolve
from .spec import stored_shapes as stored_shapes_of

SINGLE = "model.safetensors"
INDEX = "model.safetensors.index.json"
COMPUTE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def discover(folder) -> dict[str, st.TensorEntry]:
    """Headers of `model.safetensors`, or of the shards an index names."""
    folder = Path(folder)
    single, index = folder / SINGLE, folder / INDEX
    if single.is_file() and index.is_file():
        raise CheckpointError(f"{folder}: both {SINGLE} and {INDEX} are present")
    if single.is_file():
        return st.read_header(single)
    if index.is_file():
        try:
            weight_map = json.loads(index.read_text())["weight_map"]
        except (json.JSONDecodeError, KeyError, TypeError):
            raise CheckpointError(f"{index}: not a safetensors index") from None
        entries: dict[str, st.TensorEntry] = {}
        for shard in sorted(set(weight_map.values())):
            path = (folder / shard).resolve()
            if folder.resolve() not in path.parents:
                raise CheckpointError(f"{index}: shard `{shard}` leaves the model folder")
            for name, entry in st.read_header(path).items():
                if weight_map.get(name) == shard:
                    entries[name] = entry
        lost = sorted(set(weight_map) - set(entries))
        if lost:
            raise CheckpointError(f"{index}: tensors named by the index are in no shard: {lost}", missing=lost)
        return entries
    raise CheckpointError(f"{folder}: no {SINGLE} (or {INDEX}) found")


def _namespace(plan: WeightPlan, present: set[str]) -> str:
    if plan.probe is None or len(plan.namespaces) == 1:
        return plan.namespaces[0]
    hits = [ns for ns in plan.namespaces if ns + plan.probe in present]
    if len(hits) != 1:
        names = [ns + plan.probe for ns in plan.namespaces]
        raise CheckpointError(f"cannot tell the checkpoint's namespace: exactly one of {names} must be present, "
                              f"found {len(hits)}")
    return hits[0]


def check(plan: WeightPlan, entries: dict[str, st.TensorEntry]) -> tuple[str, dict[str, st.TensorEntry]]:
    """Compares the file's tensors with the plan; raises one error that lists every difference."""
    prefix = _namespace(plan, set(entries))
    local = {}
    outside = []
    for name, entry in entries.items():
        if name.startswith(prefix):
            local[name[len(prefix):]] = entry
        else:
            outside.append(name)
    wanted = plan.stored()        # (stored name -> shape and kind: the model's tensors seen through their sources)
    missing = sorted(n for n in wanted if n not in local)
    unexpected = sorted(n for n in local if n not in wanted and n not in plan.ignored and n not in plan.tied)
    # names outside the namespace are unexpected unless they are a tied alias (lm_head.weight next to transformer.*)
    unexpected += sorted(n for n in outside if n not in plan.tied)
    mismatched = []
    for name, spec in wanted.items():
        entry = local.get(name)
        if entry is None:
            continue
        if tuple(entry.shape) != tuple(spec.shape):
            mismatched.append(f"{name}: expected shape {list(spec.shape)}, found {list(entry.shape)}")
        elif spec.kind in (MATRIX, VECTOR) and not entry.is_float:
            mismatched.append(f"{name}: expected a float dtype, found {entry.dtype}")
        elif spec.kind == TABLE and entry.is_float:
            mismatched.append(f"{name}: expected an integer dtype, found {entry.dtype}")
    tied_entries = {}
    for alias, target in plan.tied.items():
        entry = local.get(alias) or entries.get(alias)
        if entry is None or target not in local:
            continue
        other = local[target]
        if tuple(entry.shape) != tuple(other.shape) or entry.dtype != other.dtype:
            mismatched.append(f"{alias}: tied to {target} but has shape {list(entry.shape)} {entry.dtype}, "
                              f"not {list(other.shape)} {other.dtype}")
        else:
            tied_entries[alias] = (entry, other)
    mismatched.sort()
    if missing or unexpected or mismatched:
        parts = []
        if missing:
            parts.append(f"missing tensors ({len(missing)}): {missing}")
        if unexpected:
            parts.append(f"unexpected tensors ({len(unexpected)}): {unexpected}")
        if mismatched:
            parts.append(f"wrong shape or dtype ({len(mismatched)}): {mismatched}")
        raise CheckpointError("checkpoint does not match the model: " + "; ".join(parts),
                              missing=missing, unexpected=unexpected, mismatched=mismatched)
    for alias, (entry, other) in tied_entries.items():
        if st.read_raw(entry) != st.read_raw(other):
            raise CheckpointError(f"tied tensor `{alias}` differs from `{plan.tied[alias]}`",
                                  mismatched=[f"{alias}: bytes differ from {plan.tied[alias]}"])
    return prefix, {name: local[name] for name in wanted}


def keep_dtype(kind: str, compute_dtype: torch.dtype) -> torch.dtype:
    """Matrices and embedding tables take the compute dtype (rounded once, to nearest even,
    when it is bfloat16); gains, shifts and biases are 32-bit on every path; integer tables int32."""
    if kind == TABLE:
        return torch.int32
    if kind == VECTOR:
        return torch.float32
    return compute_dtype


def load_weights(folder, plan: WeightPlan, dtype: str, device) -> tuple[dict[str, torch.Tensor], list[dict]]:
    """Returns the tensors of `plan` on `device`, plus a report (name, shape, stored dtype, kept dtype, bytes)."""
    if dtype not in COMPUTE_DTYPES:
        raise CheckpointError(f"dtype must be one of {sorted(COMPUTE_DTYPES)}, found `{dtype}`")
    compute = COMPUTE_DTYPES[dtype]
    _, entries = check(plan, discover(folder))
    stored_host: dict[str, torch.Tensor] = {}
    tensors, report = {}, []
    for name, spec in plan.tensors.items():
        source = plan.source_of(name)
        target = keep_dtype(spec.kind, compute)
        if isinstance(source, Stored) and not source.transposed:
            host = st.read_tensor(entries[source.name])          # (read, used and dropped: one tensor at a time)
            action = "map"
        else:
            for stored_name, _ in stored_shapes_of(source, spec.shape):
                if stored_name not in stored_host:
                    stored_host[stored_name] = st.read_tensor(entries[stored_name])
            host = resolve(source, stored_host)
            action = type(source).__name__.lower() if not isinstance(source, Stored) else "transpose"
        kept = host.to(target).contiguous().to(device)
        if tuple(kept.shape) != tuple(spec.shape):
            raise CheckpointError(f"{name}: its source makes shape {list(kept.shape)}, the model wants {list(spec.shape)}")
        tensors[name] = kept
        stored_dtypes = sorted({entries[n].dtype for n, _ in stored_shapes_of(source, spec.shape)})
        report.append(dict(name=name, shape=list(spec.shape), stored="/".join(stored_dtypes),
                           kept=str(target).replace("torch.", ""), bytes=kept.numel() * kept.element_size(),
                           action=action))
    return tensors, report
