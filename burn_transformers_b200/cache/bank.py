"""The cache of one engine: a slot per live sequence, pages of keys and values per group of
layers, fixed-size state per sequence.

Layer calls with the same key/value needs (heads, head size, window) form a group with a page
pool of its own, `k[layer][page][kv_head][PAGE_SIZE][head_dim]`; a sequence holds one page per
64 positions in every group (a windowed group cycles through as many pages as its window spans),
so one page id addresses the same rows in every layer of the group.  This mirrors the reference's
bank of homogeneous cache groups (src/cache/tensor/state.rs:36-60, src/cache/tensor/kv.rs:65-86 of
NoahIsCool/burn-transformers) with pages in place of its dense [batch, heads, time, head_dim] planes.

Lengths advance only when a step is committed; a step that fails leaves them unchanged
(src/cache/tensor/state/step.rs:1-56).  Releasing a slot returns its pages and zeroes its state.

The tensors live here; the books (which slot and page is in use, each sequence's page list and length) are kept by the
host library, csrc/host/page_book.cpp, in C++.
"""
from __future__ import annotations

import ctypes
import dataclasses

import torch

from ..errors import CacheError
from . import native
from .spec import PAGE_SIZE, CacheConfig, CacheNeed, KvSpec


def pages_for(tokens: int) -> int:
    return (tokens + PAGE_SIZE - 1) // PAGE_SIZE


class _SlotBooks:
    """The slots of a bank as the host library keeps them: how many are free or held, whether one is held."""

    def __init__(self, bank):
        self._bank = bank
        self.count = bank.config.max_slots

    @property
    def free(self) -> int:
        return self._bank._lib.bth_book_free_slots(self._bank._book)

    @property
    def held(self) -> int:
        return self.count - self.free

    def is_held(self, slot: int) -> bool:
        return bool(self._bank._lib.bth_book_slot_is_held(self._bank._book, int(slot)))


class _PageBooks:
    """The page pool of one group as the host library keeps it."""

    def __init__(self, bank, group: int, count: int):
        self._bank, self._group, self.count = bank, group, count

    @property
    def free(self) -> int:
        return self._bank._lib.bth_book_free_pages(self._bank._book, self._group)

    @property
    def held(self) -> int:
        return self.count - self.free


@dataclasses.dataclass
class KvGroup:
    spec: KvSpec
    entries: list[int]            # cache entry ids, in layer order inside the group
    table_len: int                # pages a sequence may hold (all keys) or cycles through (window)
    pool: _PageBooks
    k: torch.Tensor               # [layers, pages, kv_heads, PAGE_SIZE, head_dim]
    v: torch.Tensor

    @property
    def is_ring(self) -> bool:
        return self.spec.window is not None


class CacheBank:
    """The tensors of the cache (pages of keys and values per group, fixed-size states) and, through the host
    library (csrc/host/page_book.cpp), its books: slots, pages, page lists and lengths."""

    def __init__(self, needs: list[CacheNeed], config: CacheConfig, kv_dtype: torch.dtype, device):
        self.config = config
        self.device = torch.device(device)
        self.kv_dtype = kv_dtype
        self.table_width = pages_for(config.max_context)
        self.groups: list[KvGroup] = []
        self._entry_group: dict[int, tuple[int, int]] = {}
        self.states: dict[tuple[int, str], torch.Tensor] = {}
        self._lib = native.library()
        self._book = None
        budget_pages = pages_for(config.max_tokens)
        by_spec: dict[KvSpec, list[int]] = {}
        for entry, need in enumerate(needs):
            if need.kv is not None:
                by_spec.setdefault(need.kv, []).append(entry)
            for state in need.states:
                self.states[(entry, state.name)] = torch.zeros((config.max_slots, *state.shape), dtype=state.dtype,
                                                               device=self.device)
        table_lens, pool_sizes = [], []
        for spec, entries in by_spec.items():
            if spec.window is None:
                table_len, n_pages = self.table_width, budget_pages
            else:
                table_len = min(self.table_width, pages_for(spec.window))
                n_pages = min(budget_pages, config.max_slots * table_len)
            shape = (len(entries), n_pages, spec.n_kv_heads, PAGE_SIZE, spec.head_dim)
            group = KvGroup(spec, entries, table_len, _PageBooks(self, len(self.groups), n_pages),
                            torch.zeros(shape, dtype=kv_dtype, device=self.device),
                            torch.zeros(shape, dtype=kv_dtype, device=self.device))
            for layer, entry in enumerate(entries):
                self._entry_group[entry] = (len(self.groups), layer)
            self.groups.append(group)
            table_lens.append(table_len)
            pool_sizes.append(n_pages)
        n = len(self.groups)
        self._book = self._lib.bth_book_create(config.max_slots, config.max_context, config.max_tokens, n,
                                               (ctypes.c_int * max(1, n))(*table_lens),
                                               (ctypes.c_int * max(1, n))(*pool_sizes))
        if not self._book:
            raise native.error()
        self.slots = _SlotBooks(self)
        self._row = (ctypes.c_int * max(1, self.table_width))()

    def __del__(self):
        book, self._book = getattr(self, "_book", None), None
        if book:
            self._lib.bth_book_destroy(book)

    @property
    def max_continued_run(self) -> int | None:
        """The most tokens one step may add to a sequence that already holds some; None: no limit.

        A windowed group keeps a ring of `table_len` pages.  The step's keys are filed before its queries attend, so
        the newest token's key must not overwrite a key the step's first token still sees: a run of n tokens is
        safe while n <= ring - window + 1.  Groups that keep every key have no such limit."""
        runs = [g.table_len * PAGE_SIZE - g.spec.window + 1 for g in self.groups if g.is_ring]
        return max(1, min(runs)) if runs else None

    # ---- slots -------------------------------------------------------------------------
    def acquire(self) -> int:
        slot = self._lib.bth_book_acquire(self._book)
        if slot < 0:
            raise native.error()
        return slot

    def release(self, slot: int) -> None:
        if self._lib.bth_book_release(self._book, int(slot)) < 0:
            raise native.error()
        for state in self.states.values():
            state[slot].zero_()

    def length(self, slot: int) -> int:
        n = self._lib.bth_book_length(self._book, int(slot))
        if n < 0:
            raise native.error()
        return n

    # ---- pages -------------------------------------------------------------------------
    def reserve(self, wanted: list[tuple[int, int]]) -> None:
        """Gives every (slot, new_length) the pages it needs, or raises and changes nothing."""
        n = len(wanted)
        slots = (ctypes.c_int * max(1, n))(*[int(s) for s, _ in wanted])
        lens = (ctypes.c_int * max(1, n))(*[int(m) for _, m in wanted])
        if self._lib.bth_book_reserve(self._book, n, slots, lens) < 0:
            raise native.error()

    def commit(self, slot: int, new_len: int) -> None:
        if self._lib.bth_book_commit(self._book, int(slot), int(new_len)) < 0:
            raise native.error()

    def table_row(self, group_index: int, slot: int) -> list[int]:
        n = self._lib.bth_book_table_row(self._book, int(group_index), int(slot), self._row, self.table_width)
        if n < 0:
            raise native.error()
        return list(self._row[:n])

    def entry_group(self, entry: int) -> tuple[int, int]:
        """(group index, layer index inside the group) of a cache entry that holds keys and values."""
        return self._entry_group[entry]

    def layer_pools(self, entry: int) -> tuple[torch.Tensor, torch.Tensor, KvGroup, int]:
        g, layer = self._entry_group[entry]
        group = self.groups[g]
        return group.k[layer], group.v[layer], group, g

    def state(self, entry: int, name: str) -> torch.Tensor:
        return self.states[(entry, name)]

    # ---- checks ------------------------------------------------------------------------
    def tokens_held(self) -> int:
        """Tokens the live sequences hold, each rounded up to a whole page."""
        return int(self._lib.bth_book_tokens_held(self._book))

    def check(self) -> None:
        """No slot or page lost, held twice or freed twice."""
        if self._lib.bth_book_check(self._book) < 0:
            raise native.error()
