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
"""
from __future__ import annotations

import dataclasses

import torch

from ..errors import CacheError
from .slots import FreeList
from .spec import PAGE_SIZE, CacheConfig, CacheNeed, KvSpec


def pages_for(tokens: int) -> int:
    return (tokens + PAGE_SIZE - 1) // PAGE_SIZE


@dataclasses.dataclass
class KvGroup:
    spec: KvSpec
    entries: list[int]            # cache entry ids, in layer order inside the group
    table_len: int                # pages a sequence may hold (all keys) or cycles through (window)
    pool: FreeList
    k: torch.Tensor               # [layers, pages, kv_heads, PAGE_SIZE, head_dim]
    v: torch.Tensor
    pages: dict[int, list[int]]   # slot -> page ids in logical order

    @property
    def is_ring(self) -> bool:
        return self.spec.window is not None


class CacheBank:
    def __init__(self, needs: list[CacheNeed], config: CacheConfig, kv_dtype: torch.dtype, device):
        self.config = config
        self.device = torch.device(device)
        self.kv_dtype = kv_dtype
        self.slots = FreeList(config.max_slots, "slot")
        self.lengths = [0] * config.max_slots
        self.table_width = pages_for(config.max_context)
        self.groups: list[KvGroup] = []
        self._entry_group: dict[int, tuple[int, int]] = {}
        self.states: dict[tuple[int, str], torch.Tensor] = {}
        budget_pages = pages_for(config.max_tokens)
        by_spec: dict[KvSpec, list[int]] = {}
        for entry, need in enumerate(needs):
            if need.kv is not None:
                by_spec.setdefault(need.kv, []).append(entry)
            for state in need.states:
                self.states[(entry, state.name)] = torch.zeros((config.max_slots, *state.shape), dtype=state.dtype,
                                                               device=self.device)
        for spec, entries in by_spec.items():
            if spec.window is None:
                table_len, n_pages = self.table_width, budget_pages
            else:
                table_len = min(self.table_width, pages_for(spec.window))
                n_pages = min(budget_pages, config.max_slots * table_len)
            shape = (len(entries), n_pages, spec.n_kv_heads, PAGE_SIZE, spec.head_dim)
            group = KvGroup(spec, entries, table_len, FreeList(n_pages, "cache page"),
                            torch.zeros(shape, dtype=kv_dtype, device=self.device),
                            torch.zeros(shape, dtype=kv_dtype, device=self.device), {})
            for layer, entry in enumerate(entries):
                self._entry_group[entry] = (len(self.groups), layer)
            self.groups.append(group)

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
        slot = self.slots.take()
        self.lengths[slot] = 0
        for group in self.groups:
            group.pages[slot] = []
        return slot

    def release(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not in use (released twice?)")
        for group in self.groups:
            for page in group.pages.pop(slot, []):
                group.pool.give_back(page)
        for state in self.states.values():
            state[slot].zero_()
        self.lengths[slot] = 0
        self.slots.give_back(slot)

    def length(self, slot: int) -> int:
        self._held(slot)
        return self.lengths[slot]

    def _held(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not in use")

    # ---- pages -------------------------------------------------------------------------
    def _pages_wanted(self, group: KvGroup, new_len: int) -> int:
        return min(pages_for(new_len), group.table_len)

    def reserve(self, wanted: list[tuple[int, int]]) -> None:
        """Gives every (slot, new_length) the pages it needs, or raises and changes nothing."""
        for slot, new_len in wanted:
            self._held(slot)
            if new_len > self.config.max_context:
                raise CacheError(f"slot {slot}: {new_len} tokens exceed the longest sequence of "
                                 f"{self.config.max_context}")
            if new_len < self.lengths[slot]:
                raise CacheError(f"slot {slot}: cannot shrink from {self.lengths[slot]} to {new_len} tokens")
        for group in self.groups:
            extra = sum(max(0, self._pages_wanted(group, n) - len(group.pages[s])) for s, n in wanted)
            if extra > group.pool.free:
                raise CacheError(f"the cache is full: {extra} more pages needed, {group.pool.free} of "
                                 f"{group.pool.count} free (max_tokens={self.config.max_tokens})")
        for group in self.groups:
            for slot, new_len in wanted:
                held = group.pages[slot]
                held.extend(group.pool.take_many(max(0, self._pages_wanted(group, new_len) - len(held))))

    def commit(self, slot: int, new_len: int) -> None:
        self._held(slot)
        self.lengths[slot] = new_len

    def table_row(self, group_index: int, slot: int) -> list[int]:
        return self.groups[group_index].pages[slot]

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
        return sum(pages_for(self.lengths[s]) * PAGE_SIZE for s in range(self.config.max_slots) if self.slots.is_held(s))

    def check(self) -> None:
        """No slot or page lost, held twice or freed twice."""
        self.slots.check()
        for group in self.groups:
            group.pool.check()
            held = [p for pages in group.pages.values() for p in pages]
            if len(held) != len(set(held)):
                raise CacheError("a cache page is held by two sequences")
            if len(held) != group.pool.held:
                raise CacheError("cache pages are lost: held pages and page lists differ")
            if any(not self.slots.is_held(s) for s in group.pages):
                raise CacheError("a free slot still holds pages")
