"""Replays token sequences through the engine under different schedules and collects the logits
per (request, position), for comparison with the plain implementation."""
from __future__ import annotations

import numpy as np

from burn_transformers_b200 import Engine, StepEntry


def _take(store, logits, wanted):
    host = logits.detach().cpu().double().numpy()
    assert host.shape[0] == len(wanted)
    for row, key in zip(host, wanted):
        store[key] = row


def whole(engine: Engine, seqs):
    """Each request alone, all of it in one step."""
    got = {}
    for r, seq in enumerate(seqs):
        slot = engine.new_sequence()
        _take(got, engine.step([StepEntry(slot, seq, list(range(len(seq))))]), [(r, p) for p in range(len(seq))])
        engine.release(slot)
    return got


def tail_one_by_one(engine: Engine, seqs, tail=32):
    """Each request alone: all but the last `tail` tokens in one step, then one token a step."""
    got = {}
    for r, seq in enumerate(seqs):
        slot = engine.new_sequence()
        head = max(1, len(seq) - tail)
        _take(got, engine.step([StepEntry(slot, seq[:head], list(range(head)))]), [(r, p) for p in range(head)])
        for p in range(head, len(seq)):
            _take(got, engine.step([StepEntry(slot, [seq[p]], [0])]), [(r, p)])
        engine.release(slot)
    return got


def batches(engine: Engine, seqs, groups, prompt_lengths):
    """Batches that start together with unequal prompts, then one token each; a request leaves when its
    tokens are used up; one batch after another on the same engine."""
    got = {}
    for group in groups:
        slots = {r: engine.new_sequence() for r in group}
        entries, wanted = [], []
        for r in group:
            n = prompt_lengths[r]
            entries.append(StepEntry(slots[r], seqs[r][:n], list(range(n))))
            wanted += [(r, p) for p in range(n)]
        _take(got, engine.step(entries), wanted)
        fed = {r: prompt_lengths[r] for r in group}
        while True:
            live = [r for r in group if fed[r] < len(seqs[r])]
            if not live:
                break
            _take(got, engine.step([StepEntry(slots[r], [seqs[r][fed[r]]], [0]) for r in live]),
                  [(r, fed[r]) for r in live])
            for r in live:
                fed[r] += 1
        for r in group:
            engine.release(slots[r])
        engine.cache.check()
    return got


def worst_error(got, reference_logits):
    """Largest |difference| over all positions, relative to the largest |reference logit| of its row's sequence."""
    worst, where = 0.0, None
    for (r, p), row in got.items():
        ref = reference_logits[r][p]
        err = float(np.abs(row - ref).max() / np.abs(reference_logits[r]).max())
        if err > worst:
            worst, where = err, (r, p)
    return worst, where
