"""Replaying a given trace of steps through the model (used by ``bin/trace_run``).

The replayer keeps, per request id, its slot and how many tokens it has run; it makes
pages for what a step brings, calls the model's step function with exactly the
entries of the step, gives back pages that windows have passed, and frees requests
that the step ends.  It samples nothing.
"""
from __future__ import annotations

import torch

from ..errors import ModelError
from .model import load_model
from .step import StepEntry


class Replayer:
    def __init__(self, model_dir, *, dtype="bfloat16", max_tokens, page_size=64, max_requests=8,
                 device="cuda:0", ops=None, model=None):
        if page_size <= 0 or 64 % page_size:
            raise ModelError(f"--page-size must divide 64, got {page_size}")
        n_pages = max(1, -(-int(max_tokens) // page_size))
        self.model = model or load_model(model_dir, dtype=dtype, device=device, ops=ops, page_size=page_size,
                                         n_pages=n_pages, max_slots=max_requests,
                                         max_step_tokens=max(int(max_tokens), 64))
        self.live = {}      # request id -> [slot, tokens run]

    def run_step(self, entries, end=(), record=None):
        """entries: [{"id", "tokens", "want"}]; returns CPU float32 logits [wanted, vocab] or None.
        ``record``: a dict that parts fill with internals of this step (tests)."""
        m = self.model
        batch = []
        for e in entries:
            rid, tokens = e["id"], list(e["tokens"])
            if not tokens:
                continue
            if rid not in self.live:
                self.live[rid] = [m.cache.admit(), 0]
            slot, done = self.live[rid]
            m.cache.ensure(slot, done, done + len(tokens))
            batch.append(StepEntry(slot, done, tokens, list(e.get("want", []))))
        logits = None
        if batch:
            out = m.step(batch, record=record)
            for b in batch:
                rec = next(v for v in self.live.values() if v[0] == b.slot)
                rec[1] += len(b.tokens)
                m.cache.advance(b.slot, rec[1])
            if out.shape[0]:
                logits = out.to("cpu", torch.float32)
            m.check_status()
        for rid in end:
            if rid in self.live:
                m.cache.release(self.live.pop(rid)[0])
        return logits
