"""The scheduler: which requests run in the next step, with how many tokens each.

Decisions, in order, every step (deterministic, by arrival):
  1. every running request that has one token left to run (decoding) takes that token;
  2. running requests that still have prompt left take a portion of it, limited by
     ``prefill_chunk`` and by what is left of the step's token budget;
  3. waiting requests are admitted first-come first-served while a request slot, budget
     and pages for their first portion are there.
When pages run out for a request that is already running, the request that arrived
last among the running ones is preempted: its pages and slot are given back, it goes
to the front of the waiting queue and is later recomputed from its prompt and the
tokens it has generated so far.  A request that can never fit (longer than the context
limit, or needing more pages than the pool has) fails alone, with an error.

The reference fills a step of at most 128 tokens by walking its sessions, gives a
prefilling session what is left of the budget, reserves all pages of a prompt at
creation, has no waiting queue and no preemption: a failed page allocation aborts the
step for everyone (crates/thuban_generate/src/engine.rs:103-300).  This file needs no
device: it sees the cache manager only through ``can_run / ensure / advance / admit /
release / free_slots``.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from ..errors import CacheError
from ..sampling.params import SamplingParams, SplitMix64

WAITING, RUNNING, FINISHED, FAILED = "waiting", "running", "finished", "failed"


@dataclass(eq=False)
class Request:
    id: int
    prompt: list
    max_tokens: int
    sampling: SamplingParams
    stop: tuple
    rng: SplitMix64
    arrival: int
    generated: list = field(default_factory=list)
    state: str = WAITING
    slot: int = -1
    n_cached: int = 0          # tokens whose keys and values are in the cache
    error: str | None = None
    finish_reason: str | None = None
    preemptions: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0

    @property
    def tokens(self):
        return self.prompt + self.generated

    @property
    def n_tokens(self):
        return len(self.prompt) + len(self.generated)

    def span(self, start, n):
        """Tokens [start, start + n) of prompt and generated text, without joining the two lists."""
        np_ = len(self.prompt)
        if start + n <= np_:
            return self.prompt[start:start + n]
        if start >= np_:
            return self.generated[start - np_:start - np_ + n]
        return self.prompt[start:] + self.generated[:start + n - np_]

    @property
    def remaining(self):
        return len(self.prompt) + len(self.generated) - self.n_cached


@dataclass
class Portion:
    request: Request
    start: int
    n_tokens: int
    wants_logits: bool


class Scheduler:
    def __init__(self, cache, *, max_step_tokens=8192, prefill_chunk=2048, max_context=None, total_pages=None,
                 page_size=None):
        self.cache = cache
        self.max_step_tokens = int(max_step_tokens)
        self.prefill_chunk = int(prefill_chunk)
        self.max_context = int(max_context if max_context is not None else cache.max_context)
        self.page_size = int(page_size if page_size is not None else cache.page_size)
        self.total_pages = int(total_pages if total_pages is not None else
                               min(g.pages.pool.n_pages for g in cache.groups) if cache.groups else 1 << 30)
        self.waiting: deque = deque()
        self.running: list = []
        self.preemptions = 0
        self.steps = 0

    # ------------------------------------------------------------------ admission
    def add(self, req: Request):
        if not req.prompt:
            self._fail(req, "empty prompt")
            return
        if len(req.prompt) + 1 > self.max_context:
            self._fail(req, f"prompt of {len(req.prompt)} tokens does not fit the context limit {self.max_context}")
            return
        req.state = WAITING
        self.waiting.append(req)

    def _fail(self, req, msg):
        req.state, req.error, req.finish_reason = FAILED, msg, "error"

    def has_work(self):
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ planning
    def _preempt(self, victim):
        """Give back the pages and the slot of a running request; it will be recomputed."""
        self.running.remove(victim)
        self.cache.release(victim.slot)
        victim.slot, victim.n_cached, victim.state = -1, 0, WAITING
        victim.preemptions += 1
        self.preemptions += 1
        self.waiting.appendleft(victim)

    def _fits_portion(self, req, n):
        """Largest m <= n such that pages exist for positions [n_cached, n_cached + m)."""
        while n > 0 and not self.cache.can_run(req.slot, req.n_cached, req.n_cached + n):
            n = (n - 1) // self.page_size * self.page_size if n > self.page_size else n - 1
        return n

    def _make_room(self, req, portions, planned):
        """Pages ran out for ``req``: preempt running requests that arrived after it, the
        last one first, until at least one token of ``req`` fits.  Returns the budget
        given back by voided portions.  If nobody younger is left, ``req`` itself is
        preempted (others are older and go first), or fails if it is alone."""
        refund = 0
        while req in self.running and not self.cache.can_run(req.slot, req.n_cached, req.n_cached + 1):
            younger = [r for r in self.running if r.arrival > req.arrival]
            if younger:
                victim = max(younger, key=lambda r: r.arrival)
            elif len(self.running) == 1:
                self.running.remove(req)
                self.cache.release(req.slot)
                req.slot = -1
                self._fail(req, f"request of {req.n_tokens} tokens needs more pages than the pool has")
                break
            else:
                victim = req
            if victim in planned:
                for p in [p for p in portions if p.request is victim]:
                    refund += p.n_tokens
                    portions.remove(p)
                planned.discard(victim)
            self._preempt(victim)
        return refund

    def plan(self):
        """Returns the list of Portions of the next step (their pages are made)."""
        budget = self.max_step_tokens
        portions, planned = [], set()
        # 1. decoding requests, then 2. running requests with prompt (or recomputation) left;
        #    each oldest first
        for decoding in (True, False):
            for req in sorted(self.running, key=lambda r: r.arrival):
                if req not in self.running or req in planned or budget <= 0 or req.remaining < 1:
                    continue
                if decoding != (req.remaining == 1):
                    continue
                n = self._fits_portion(req, min(req.remaining, self.prefill_chunk, budget))
                if n == 0:
                    budget += self._make_room(req, portions, planned)
                    if req not in self.running:
                        continue
                    n = self._fits_portion(req, min(req.remaining, self.prefill_chunk, budget))
                    if n == 0:
                        continue
                self.cache.ensure(req.slot, req.n_cached, req.n_cached + n)
                portions.append(Portion(req, req.n_cached, n, n == req.remaining))
                planned.add(req)
                budget -= n
        # 3. admit waiting requests, first come first served; never preempts
        while self.waiting and budget > 0 and self.cache.free_slots > 0:
            req = self.waiting[0]
            need_pages = -(-req.n_tokens // self.page_size)
            if req.n_tokens + 1 > self.max_context or (need_pages > self.total_pages and not self._windowed()):
                self.waiting.popleft()
                self._fail(req, f"request of {req.n_tokens} tokens can never fit "
                                f"({self.total_pages} pages of {self.page_size}, context limit {self.max_context})")
                continue
            slot = self.cache.admit()
            req.slot = slot
            n = self._fits_portion(req, min(req.remaining, self.prefill_chunk, budget))
            if n == 0:
                self.cache.release(slot)
                req.slot = -1
                break                            # no pages now; it keeps its place at the head
            self.waiting.popleft()
            req.state = RUNNING
            self.running.append(req)
            self.cache.ensure(slot, req.n_cached, req.n_cached + n)
            portions.append(Portion(req, req.n_cached, n, n == req.remaining))
            planned.add(req)
            budget -= n
        self.steps += 1
        return portions

    def _windowed(self):
        return any(g.pages.window for g in self.cache.groups) if getattr(self.cache, "groups", None) else False

    # ------------------------------------------------------------------ after the step
    def commit(self, portions, sampled):
        """``sampled``: one token per portion that wanted logits, in order.  Returns the
        list of (request, token) emitted in this step."""
        emitted = []
        it = iter(sampled)
        for p in portions:
            req = p.request
            if p.n_tokens == 1 and p.start >= len(req.prompt):
                req.decode_tokens += 1
            else:
                req.prefill_tokens += p.n_tokens
            req.n_cached = p.start + p.n_tokens
            self.cache.advance(req.slot, req.n_cached)
            if not p.wants_logits:
                continue
            token = int(next(it))
            if token in req.stop:
                self._finish(req, "stop")
                continue
            req.generated.append(token)
            emitted.append((req, token))
            if len(req.generated) >= req.max_tokens:
                self._finish(req, "length")
            elif req.n_tokens + 1 > self.max_context:
                self._finish(req, "context")
        return emitted

    def _finish(self, req, reason):
        req.state, req.finish_reason = FINISHED, reason
        if req in self.running:
            self.running.remove(req)
        if req.slot >= 0:
            self.cache.release(req.slot)
            req.slot = -1

    def abort(self, req):
        if req in self.waiting:
            self.waiting.remove(req)
        self._finish(req, "abort")
