"""The packing of a step's integers (done by the host library, csrc/host/page_book.cpp) against the same packing
written out in Python: tokens, positions from the cache's lengths, sequence starts, lengths, wanted rows, page tables.
No GPU: the builder runs on the CPU device."""
import random

import torch

from burn_transformers_b200.cache import CacheBank, CacheConfig, CacheNeed, KvSpec, PAGE_SIZE
from burn_transformers_b200.engine import StepBuilder, StepEntry


def make_bank():
    needs = [CacheNeed(kv=KvSpec(2, 16)), CacheNeed(kv=KvSpec(1, 32, window=100))]
    return CacheBank(needs, CacheConfig(64 * 40, 6, 64 * 8), torch.float32, "cpu")


def expected(bank, entries):
    tokens, positions, token_seq, seq_start, past, ctx, slots, want_rows = [], [], [], [0], [], [], [], []
    for i, e in enumerate(entries):
        p = bank.length(e.slot)
        want_rows += [len(tokens) + w for w in e.want]
        tokens += list(e.tokens)
        positions += list(range(p, p + len(e.tokens)))
        token_seq += [i] * len(e.tokens)
        seq_start.append(len(tokens))
        past.append(p)
        ctx.append(p + len(e.tokens))
        slots.append(e.slot)
    tables = []
    for g in range(len(bank.groups)):
        rows = []
        for e in entries:
            row = bank.table_row(g, e.slot)
            rows.append(row + [0] * (bank.table_width - len(row)))
        tables.append(rows)
    return tokens, positions, token_seq, seq_start, past, ctx, slots, want_rows, tables


def test_packed_steps_match_the_written_out_packing():
    rng = random.Random(5)
    bank = make_bank()
    builder = StepBuilder(bank, torch.float32, "cpu")
    live = {}
    for step in range(60):
        while len(live) < 4 and rng.random() < 0.6:
            live[bank.acquire()] = 0
        if not live:
            continue
        chosen = rng.sample(sorted(live), rng.randint(1, len(live)))
        entries = []
        for slot in chosen:
            room = 64 * 8 - live[slot]
            if room <= 0:
                continue
            n = min(room, rng.choice([1, 1, 2, 7, 64, 65, 130]))
            toks = [rng.randrange(1000) for _ in range(n)]
            want = sorted(rng.sample(range(n), rng.randint(0, min(n, 3))))
            entries.append(StepEntry(slot, toks, want))
        if not entries:
            continue
        bank.reserve([(e.slot, live[e.slot] + len(e.tokens)) for e in entries])
        want = expected(bank, entries)
        ctx = builder.build(entries)
        n_tok, n_seq, n_want = len(want[0]), len(entries), len(want[7])
        assert (ctx.n_tokens, ctx.n_seqs, ctx.n_want) == (n_tok, n_seq, n_want)
        assert ctx.max_new == max(len(e.tokens) for e in entries)
        assert ctx.is_decode == all(len(e.tokens) == 1 for e in entries)
        assert ctx.fresh == all(live[e.slot] == 0 for e in entries)
        assert ctx.ctx_bound == max(want[5])
        assert ctx.tokens[:n_tok].tolist() == want[0]
        assert ctx.positions[:n_tok].tolist() == want[1]
        assert ctx.token_seq[:n_tok].tolist() == want[2]
        assert ctx.seq_start[:n_seq + 1].tolist() == want[3]
        assert ctx.past_len[:n_seq].tolist() == want[4]
        assert ctx.ctx_len[:n_seq].tolist() == want[5]
        assert ctx.slots[:n_seq].tolist() == want[6]
        assert ctx.want_rows[:n_want].tolist() == want[7]
        for g, table in enumerate(ctx.tables):
            assert table.tolist() == want[8][g]
        for e in entries:
            live[e.slot] += len(e.tokens)
            bank.commit(e.slot, live[e.slot])
        for slot in list(live):
            if rng.random() < 0.15 or live[slot] >= 64 * 8:
                bank.release(slot)
                del live[slot]
        bank.check()


def test_a_slot_that_is_not_held_is_refused_by_the_packer():
    import pytest
    from burn_transformers_b200.errors import CacheError
    bank = make_bank()
    builder = StepBuilder(bank, torch.float32, "cpu")
    slot = bank.acquire()
    bank.release(slot)
    with pytest.raises(CacheError, match="not in use"):
        builder.build([StepEntry(slot, [1, 2], [1])])
