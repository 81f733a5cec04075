"""Token selection on the device: edits, then the selection kernel, then one small copy to the host."""
from __future__ import annotations

import torch

from .. import kernels
from ..errors import GenerationError
from .config import GenerationConfig
from .random import sequence_stream, uniform


class DeviceSampler:
    """Selects one token per row of a step's logits.

    Per step the host sends: the uniforms (one float per row) and, if a penalty, bias or ban is
    active, the sparse edits; it reads back the ids and their log-probabilities.  These copies
    are the loop's only synchronisation with the device (the reference syncs once per step too,
    src/generation/causal.rs:170-172)."""

    def __init__(self, config: GenerationConfig, vocab: int, device, max_rows: int):
        config.validate(vocab)
        self.config, self.vocab, self.device = config, vocab, torch.device(device)
        self.max_rows = max_rows
        self.ids = torch.empty(max_rows, dtype=torch.int32, device=self.device)
        self.logp = torch.empty(max_rows, dtype=torch.float32, device=self.device)
        self.uniforms = torch.empty(max_rows, dtype=torch.float32, device=self.device)
        self.host_out = torch.empty(2 * max_rows, dtype=torch.int32, pin_memory=True)
        self.host_u = torch.empty(max_rows, dtype=torch.float32, pin_memory=True)
        self.reference_counter = 0
        self.d2h_bytes_last = 0
        self.h2d_bytes_last = 0

    def _uniforms(self, trackers, batch_rows: int) -> None:
        cfg = self.config
        n = len(trackers)
        if cfg.counter_mode == "reference":
            # one block of `batch_rows` counters per step; row b of the original batch uses start + b
            for i, t in enumerate(trackers):
                self.host_u[i] = uniform(cfg.seed, self.reference_counter + t.row_in_batch)
            self.reference_counter += batch_rows
        else:
            for i, t in enumerate(trackers):
                self.host_u[i] = uniform(sequence_stream(cfg.seed, t.request), t.emitted)
        self.uniforms[:n].copy_(self.host_u[:n], non_blocking=True)
        self.h2d_bytes_last += 4 * n

    def _edits(self, logits, trackers) -> None:
        rows, tokens, vals = [], [], []
        for i, t in enumerate(trackers):
            for token, v in t.edits().items():
                rows.append(i)
                tokens.append(token)
                vals.extend(v)
        if not rows:
            return
        dev = self.device
        r = torch.tensor(rows, dtype=torch.int32).to(dev)
        k = torch.tensor(tokens, dtype=torch.int32).to(dev)
        v = torch.tensor(vals, dtype=torch.float32).to(dev)
        self.h2d_bytes_last += 4 * (len(rows) * 2 + len(vals))
        kernels.logit_edits(logits, r, k, v, len(rows))

    def select(self, logits: torch.Tensor, trackers, batch_rows: int | None = None):
        """logits: [n, vocab] float32 on the device (edited in place).  Returns (ids, log_probabilities) as lists."""
        n = len(trackers)
        if logits.shape[0] < n or logits.shape[1] != self.vocab:
            raise GenerationError(f"generation.logits: expected [{n}, {self.vocab}], found {list(logits.shape)}")
        cfg = self.config
        self.h2d_bytes_last = 0
        if cfg.edits_logits:
            self._edits(logits, trackers)
        if cfg.samples:
            self._uniforms(trackers, batch_rows if batch_rows is not None else n)
        kernels.sample(logits, n, do_sample=cfg.samples, temperature=float(cfg.temperature),
                       top_k=(cfg.top_k if cfg.samples and cfg.top_k and cfg.top_k < self.vocab else 0),
                       top_p=(cfg.top_p if cfg.samples and cfg.top_p is not None else 1.0),
                       min_p=(cfg.min_p if cfg.samples and cfg.min_p is not None else 0.0),
                       uniforms=self.uniforms if cfg.samples else None, out_ids=self.ids, out_logp=self.logp)
        self.host_out[:n].copy_(self.ids[:n], non_blocking=True)
        self.host_out[self.max_rows:self.max_rows + n].copy_(self.logp[:n].view(torch.int32), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes_last = 8 * n
        ids = self.host_out[:n].tolist()
        logps = self.host_out[self.max_rows:self.max_rows + n].view(torch.float32).tolist()
        return ids, logps
