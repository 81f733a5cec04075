"""Reading and writing safetensors files without a library.

Format: an 8-byte little-endian header length, a JSON header mapping each tensor
name to {dtype, shape, data_offsets}, then the raw little-endian data.  The
header is bounded and checked before any tensor is touched, as the reference's
discovery pass does (src/checkpoint/artifact.rs:36-39, src/checkpoint/options.rs:53-113).
"""
from __future__ import annotations

import dataclasses
import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

from ..errors import CheckpointError

MAX_HEADER_BYTES = 100_000_000   # src/checkpoint/options.rs (ArtifactLimits::default)
MAX_TENSORS = 10_000_000
MAX_RANK = 32

# safetensors dtype tag -> (bytes per element, torch dtype, is float)
DTYPES = {
    "F64": (8, torch.float64, True),
    "F32": (4, torch.float32, True),
    "F16": (2, torch.float16, True),
    "BF16": (2, torch.bfloat16, True),
    "I64": (8, torch.int64, False),
    "I32": (4, torch.int32, False),
    "I16": (2, torch.int16, False),
    "I8": (1, torch.int8, False),
    "U8": (1, torch.uint8, False),
    "BOOL": (1, torch.bool, False),
}
TAG_OF = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16",
          torch.int32: "I32", torch.int64: "I64", torch.float64: "F64"}


@dataclasses.dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: tuple[int, ...]
    begin: int          # offsets relative to the start of the data section
    end: int
    file: Path
    data_start: int     # absolute offset of the data section in `file`

    @property
    def is_float(self) -> bool:
        return DTYPES[self.dtype][2]


def read_header(path) -> dict[str, TensorEntry]:
    """Checks and returns the header of one safetensors file; reads no tensor data."""
    path = Path(path)
    if not path.is_file():
        raise CheckpointError(f"checkpoint file not found: {path}")
    size = path.stat().st_size
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise CheckpointError(f"{path}: truncated file, no header length")
        (n,) = struct.unpack("<Q", head)
        if n == 0 or n > MAX_HEADER_BYTES or 8 + n > size:
            raise CheckpointError(f"{path}: invalid header length {n} for a file of {size} bytes")
        raw = f.read(n)
    try:
        header = json.loads(raw)
    except (json.JSONDecodeError, UnicodeDecodeError) as error:
        raise CheckpointError(f"{path}: header is not valid JSON: {error}") from None
    if not isinstance(header, dict):
        raise CheckpointError(f"{path}: header must be a JSON object")
    data_start = 8 + n
    data_bytes = size - data_start
    entries: dict[str, TensorEntry] = {}
    if len(header) > MAX_TENSORS:
        raise CheckpointError(f"{path}: header lists more than {MAX_TENSORS} tensors")
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        try:
            dtype, shape, (begin, end) = meta["dtype"], tuple(meta["shape"]), meta["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise CheckpointError(f"{path}: malformed header entry for `{name}`") from None
        if dtype not in DTYPES:
            raise CheckpointError(f"{path}: tensor `{name}` has unsupported dtype {dtype}")
        if len(shape) > MAX_RANK or any((not isinstance(s, int)) or s < 0 for s in shape):
            raise CheckpointError(f"{path}: tensor `{name}` has an invalid shape {list(shape)}")
        want = math.prod(shape) * DTYPES[dtype][0]
        if not (isinstance(begin, int) and isinstance(end, int)) or begin < 0 or end < begin or end - begin != want:
            raise CheckpointError(f"{path}: tensor `{name}` has invalid data offsets [{begin}, {end}) for {want} bytes")
        if end > data_bytes:
            raise CheckpointError(f"{path}: truncated file, tensor `{name}` ends at byte {end} of a "
                                  f"{data_bytes}-byte data section")
        entries[name] = TensorEntry(name, dtype, shape, begin, end, path, data_start)
    return entries


def read_tensor(entry: TensorEntry) -> torch.Tensor:
    """Reads one tensor to host memory in its stored dtype."""
    count = entry.end - entry.begin
    with open(entry.file, "rb") as f:
        f.seek(entry.data_start + entry.begin)
        raw = f.read(count)
    if len(raw) != count:
        raise CheckpointError(f"{entry.file}: truncated while reading `{entry.name}`")
    _, dtype, _ = DTYPES[entry.dtype]
    if count == 0:
        return torch.empty(entry.shape, dtype=dtype)
    flat = torch.frombuffer(bytearray(raw), dtype=dtype)
    return flat.reshape(entry.shape)


def read_raw(entry: TensorEntry) -> bytes:
    with open(entry.file, "rb") as f:
        f.seek(entry.data_start + entry.begin)
        return f.read(entry.end - entry.begin)


def write_file(path, tensors: dict[str, torch.Tensor], metadata: dict[str, str] | None = None) -> None:
    """Writes host tensors in name order; the header is padded so the data starts 8-byte aligned."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = metadata
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in TAG_OF:
            raise CheckpointError(f"cannot write tensor `{name}` of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": TAG_OF[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    raw = json.dumps(header, separators=(",", ":")).encode()
    raw += b" " * ((8 - len(raw) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes())
