"""One step of a batch: the tokens it brings, where they sit, and the scratch memory of the step."""
from __future__ import annotations

import dataclasses

import torch

from ..errors import KernelError


@dataclasses.dataclass
class StepEntry:
    """A sequence's share of a step: its slot, its next tokens, and the places among these tokens
    (0-based) whose logits are wanted."""
    slot: int
    tokens: list[int]
    want: list[int]


class Workspace:
    """Scratch memory of a step: one device buffer handed out piece by piece and reused every step."""

    def __init__(self, device, initial_bytes: int = 1 << 20):
        self.device = torch.device(device)
        self.buffer = torch.empty(initial_bytes, dtype=torch.uint8, device=self.device)
        self.offset = 0
        self.frozen = False       # set while a CUDA graph is captured or replayed: addresses must not move
        self._retired: list[torch.Tensor] = []

    def reset(self) -> None:
        self.offset = 0
        self._retired.clear()

    def take(self, shape, dtype) -> torch.Tensor:
        count = 1
        for s in shape:
            count *= int(s)
        nbytes = count * torch.empty((), dtype=dtype).element_size()
        start = (self.offset + 255) & ~255
        if start + nbytes > self.buffer.numel():
            if self.frozen:
                raise KernelError("the step's workspace would have to grow while a CUDA graph holds its address")
            # grow: earlier pieces of this step stay valid in the retired buffer
            self._retired.append(self.buffer)
            self.buffer = torch.empty(max(2 * self.buffer.numel(), start + nbytes + (1 << 20)), dtype=torch.uint8,
                                      device=self.device)
            start = 0
        self.offset = start + nbytes
        return self.buffer[start:start + nbytes].view(dtype).view(*shape)


class StepContext:
    """Everything a part may ask about the step it runs in."""

    def __init__(self, *, dtype, cache, ws, n_tokens, n_seqs, n_want, max_new, is_decode, fresh, ctx_bound,
                 tokens, positions, token_seq, seq_start, past_len, ctx_len, slots, want_rows, tables,
                 host_slots=None):
        self.dtype = dtype
        self.cache, self.ws = cache, ws
        self.n_tokens, self.n_seqs, self.n_want, self.max_new = n_tokens, n_seqs, n_want, max_new
        self.is_decode = is_decode      # every sequence brings exactly one token
        self.fresh = fresh              # every sequence starts at position 0
        self.ctx_bound = ctx_bound      # no sequence is longer than this after the step
        # int32 device tensors
        self.tokens, self.positions, self.token_seq = tokens, positions, token_seq
        self.seq_start, self.past_len, self.ctx_len, self.slots = seq_start, past_len, ctx_len, slots
        self.want_rows = want_rows
        self.tables = tables            # per cache group: [n_seqs, table_width] page ids
        self.host_slots = host_slots    # the slots as a Python list, for parts that index state on the host
