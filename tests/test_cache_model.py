"""The cache's books against a model written out in Python, driven by generated sequences of operations (no GPU).

The model knows only the rules: a full-attention group holds ceil(length / page) pages of a sequence, a windowed group
at most the pages its window spans; pages and slots come from fixed pools; a refused operation changes nothing.  After
every operation the books must agree with it: lengths, pages per sequence and group, free pages and slots, no page
in two rows, and the library's own check (no slot or page lost, held twice or freed twice).
"""
import pytest
import torch
from hypothesis import settings, strategies as st
from hypothesis.stateful import RuleBasedStateMachine, invariant, precondition, rule

from burn_transformers_b200.cache import CacheBank, CacheConfig, CacheNeed, KvSpec, StateSpec, PAGE_SIZE
from burn_transformers_b200.errors import CacheError

MAX_TOKENS, MAX_SLOTS, MAX_CONTEXT, WINDOW = 64 * 10, 4, 64 * 5, 70


def _pages(n: int) -> int:
    return -(-n // PAGE_SIZE)


class Books(RuleBasedStateMachine):
    def __init__(self):
        super().__init__()
        needs = [CacheNeed(kv=KvSpec(2, 16)), CacheNeed(kv=KvSpec(1, 32, window=WINDOW), states=(StateSpec("sum", (2,)),))]
        self.bank = CacheBank(needs, CacheConfig(MAX_TOKENS, MAX_SLOTS, MAX_CONTEXT), torch.float32, "cpu")
        self.full, self.ring = self.bank.groups
        self.ring_len = self.ring.table_len                      # pages a window spans
        self.pool = [g.pool.free for g in self.bank.groups]      # pages each group's pool starts with
        self.live: dict[int, int] = {}                           # slot -> committed length
        self.reserved: dict[int, int] = {}                       # slot -> length its pages reach

    def _held(self, group: int, reached: int) -> int:
        return _pages(reached) if group == 0 else min(_pages(reached), self.ring_len)

    @precondition(lambda self: len(self.live) < MAX_SLOTS)
    @rule()
    def acquire(self):
        slot = self.bank.acquire()
        assert slot not in self.live
        self.live[slot], self.reserved[slot] = 0, 0

    @precondition(lambda self: len(self.live) == MAX_SLOTS)
    @rule()
    def acquire_when_full(self):
        with pytest.raises(CacheError, match="no free slot"):
            self.bank.acquire()

    @precondition(lambda self: self.live)
    @rule(data=st.data(), grow=st.sampled_from([1, 1, 2, 17, 63, 64, 65, 130, 400]))
    def reserve_and_commit(self, data, grow):
        slot = data.draw(st.sampled_from(sorted(self.live)))
        want = self.reserved[slot] + grow
        extra = [self._held(g, want) - self._held(g, self.reserved[slot]) for g in (0, 1)]
        free = [self.pool[g] - sum(self._held(g, r) for r in self.reserved.values()) for g in (0, 1)]
        if want > MAX_CONTEXT:
            with pytest.raises(CacheError, match="exceed the longest sequence"):
                self.bank.reserve([(slot, want)])
        elif any(e > f for e, f in zip(extra, free)):
            with pytest.raises(CacheError, match="cache is full"):
                self.bank.reserve([(slot, want)])
        else:
            self.bank.reserve([(slot, want)])
            self.reserved[slot] = want
            upto = data.draw(st.integers(self.live[slot], want))          # a step may use fewer positions than it reserved
            self.bank.commit(slot, upto)
            self.live[slot] = upto

    @precondition(lambda self: len(self.live) >= 2)
    @rule(data=st.data())
    def reserve_two_at_once_or_neither(self, data):
        a, b = data.draw(st.lists(st.sampled_from(sorted(self.live)), min_size=2, max_size=2, unique=True))
        wants = {s: min(MAX_CONTEXT, self.reserved[s] + data.draw(st.sampled_from([1, 64, 129]))) for s in (a, b)}
        extra = [sum(self._held(g, wants[s]) - self._held(g, self.reserved[s]) for s in (a, b)) for g in (0, 1)]
        free = [self.pool[g] - sum(self._held(g, r) for r in self.reserved.values()) for g in (0, 1)]
        before = {s: [list(self.bank.table_row(g, s)) for g in (0, 1)] for s in self.live}
        if any(e > f for e, f in zip(extra, free)):
            with pytest.raises(CacheError, match="cache is full"):
                self.bank.reserve([(a, wants[a]), (b, wants[b])])
            assert before == {s: [list(self.bank.table_row(g, s)) for g in (0, 1)] for s in self.live}
        else:
            self.bank.reserve([(a, wants[a]), (b, wants[b])])
            self.reserved.update(wants)

    @precondition(lambda self: self.live)
    @rule(data=st.data())
    def shrinking_is_refused(self, data):
        slot = data.draw(st.sampled_from(sorted(self.live)))
        if self.live[slot] > 0:
            with pytest.raises(CacheError, match="cannot shrink"):
                self.bank.reserve([(slot, self.live[slot] - 1)])

    @precondition(lambda self: self.live)
    @rule(data=st.data())
    def release(self, data):
        slot = data.draw(st.sampled_from(sorted(self.live)))
        self.bank.state(1, "sum")[slot] = 3.0
        self.bank.release(slot)
        assert float(self.bank.state(1, "sum")[slot].abs().sum()) == 0.0
        del self.live[slot], self.reserved[slot]
        with pytest.raises(CacheError, match="released twice"):
            self.bank.release(slot)

    @invariant()
    def the_books_agree_with_the_model(self):
        self.bank.check()
        assert self.bank.slots.free == MAX_SLOTS - len(self.live)
        for g in (0, 1):
            rows = {s: list(self.bank.table_row(g, s)) for s in self.live}
            for s, row in rows.items():
                assert len(row) == self._held(g, self.reserved[s]), (g, s, row, self.reserved[s])
            pages = [p for row in rows.values() for p in row]
            assert len(pages) == len(set(pages)), "a page stands in two rows"
            assert self.bank.groups[g].pool.free == self.pool[g] - len(pages)
        for s, n in self.live.items():
            assert self.bank.length(s) == n
        assert self.bank.tokens_held() == sum(_pages(n) * PAGE_SIZE for n in self.live.values())


Books.TestCase.settings = settings(max_examples=40, stateful_step_count=40, deadline=None)
test_the_books_follow_the_model = Books.TestCase
