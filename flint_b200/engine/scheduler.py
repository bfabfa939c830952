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
step for everyone (crates/thuban_generate/src/engine.rs:103-300).

The decisions are taken by the native runtime (``csrc/host/runtime.cpp``), on the cache
manager's native bookkeeping; ``Scheduler`` here is its Python face and keeps the
``Request`` objects that callers hold in step with it.  Nothing here needs a device.
"""
from __future__ import annotations

from ctypes import c_int, byref
from dataclasses import dataclass, field

from ..csrc import runtime as rt
from ..sampling.params import SamplingParams, SplitMix64

WAITING, RUNNING, FINISHED, FAILED = "waiting", "running", "finished", "failed"
UNREAD = -1        # a sampled token that was committed before the host has read its value


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
    n_unread: int = 0          # the last n_unread entries of ``generated`` are placeholders (UNREAD)

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
    _STATES = (WAITING, RUNNING, FINISHED, FAILED)
    _REASONS = (None, "stop", "length", "context", "abort", "error")

    def __init__(self, cache, *, max_step_tokens=8192, prefill_chunk=2048, max_context=None, total_pages=None,
                 page_size=None):
        self.cache = cache
        self.max_step_tokens = int(max_step_tokens)
        self.prefill_chunk = int(prefill_chunk)
        self.max_context = int(max_context if max_context is not None else cache.max_context)
        self.page_size = int(page_size if page_size is not None else cache.page_size)
        self.total_pages = int(total_pages if total_pages is not None else
                               min(g.pages.pool.n_pages for g in cache.groups) if cache.groups else 1 << 30)
        self._lib = rt.lib()
        self._h = self._lib.flint_rt_sched_create(cache.core, self.max_step_tokens, self.prefill_chunk, self.max_context,
                                                  self.page_size, self.total_pages)
        self._reqs: dict = {}                       # native handle -> Request
        self.keep_ended = 4096                      # ended requests are forgotten when more than this many are known
        self._out = (c_int * (4 * (self.max_step_tokens + 1)))()
        self._fields = (c_int * 8)()

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.flint_rt_sched_destroy(self._h)
            self._h = None

    # ------------------------------------------------------------------ the requests' mirrors
    def _pull(self, req: Request):
        """Bring a Request in step with its native record."""
        f = self._fields
        self._lib.flint_rt_sched_request(self._h, req._handle, f)
        _, req.n_cached, req.slot, state, reason, req.preemptions, req.prefill_tokens, req.decode_tokens = f
        req.state = self._STATES[state]
        req.finish_reason = self._REASONS[reason]
        if req.state == FAILED and req.error is None:
            req.error = (self._lib.flint_rt_sched_request_error(self._h, req._handle) or b"").decode()

    def _push_stop(self, req: Request):
        stop = tuple(int(t) for t in req.stop)
        if stop != req._stop_pushed:
            self._lib.flint_rt_sched_set_stop(self._h, req._handle, rt.ints(stop), len(stop))
            req._stop_pushed = stop

    def _list(self, which):
        n = self._lib.flint_rt_sched_list(self._h, which, self._out, len(self._out))
        if n > len(self._out):                      # a queue longer than the buffer: take a larger one
            self._out = (c_int * (2 * n))()
            n = self._lib.flint_rt_sched_list(self._h, which, self._out, len(self._out))
        return [self._reqs[h] for h in self._out[:n]]

    @property
    def waiting(self) -> list:
        """The waiting requests in queue order."""
        return self._list(0)

    @property
    def running(self) -> list:
        return self._list(1)

    @property
    def preemptions(self) -> int:
        a, b = c_int(), c_int()
        self._lib.flint_rt_sched_counters(self._h, byref(a), byref(b))
        return a.value

    @property
    def steps(self) -> int:
        a, b = c_int(), c_int()
        self._lib.flint_rt_sched_counters(self._h, byref(a), byref(b))
        return b.value

    # ------------------------------------------------------------------ admission
    def add(self, req: Request):
        stop = tuple(int(t) for t in req.stop)
        req._handle = self._lib.flint_rt_sched_add(self._h, len(req.prompt), int(req.max_tokens), int(req.arrival),
                                                   rt.ints(stop), len(stop))
        req._stop_pushed = stop
        self._reqs[req._handle] = req
        self._pull(req)

    def has_work(self):
        return bool(self._lib.flint_rt_sched_has_work(self._h))

    # ------------------------------------------------------------------ planning
    def plan(self):
        """Returns the list of Portions of the next step (their pages are made)."""
        n = rt.checked(self._lib.flint_rt_sched_plan(self._h, self._out, len(self._out) // 4))
        out = self._out
        portions = [Portion(self._reqs[out[4 * i]], out[4 * i + 1], out[4 * i + 2], bool(out[4 * i + 3])) for i in range(n)]
        self._pull_touched()                        # preempted or failed
        for p in portions:                          # admitted or just planned
            self._pull(p.request)
            # A portion that starts at position 0 belongs to a request that was admitted in this plan, for the
            # first time or again after a preemption (possibly in this same plan, and possibly into the slot it
            # had before): its fixed-size state starts from zero.  The slot alone cannot tell.
            if p.start == 0 and self.cache.state:
                self.cache.reset_state(p.request.slot)
        return portions

    def _pull_touched(self):
        n = min(self._lib.flint_rt_sched_take_touched(self._h, self._out, len(self._out)), len(self._out))
        for h in set(self._out[:n]):
            req = self._reqs.get(h)            # a request that ended long ago may have been forgotten
            if req is not None:
                self._pull(req)

    # ------------------------------------------------------------------ after the step
    def commit(self, portions, sampled):
        """``sampled``: one token per portion that wanted logits, in order; ``UNREAD`` for a token whose
        value is still on the device (everything but the stop set is decided without it; ``resolve``
        brings the value later).  Returns the list of (request, token) emitted in this step."""
        flat = []
        for p in portions:
            self._push_stop(p.request)
            flat += (p.request._handle, p.start, p.n_tokens, 1 if p.wants_logits else 0)
        tokens = [int(t) for t in sampled]
        emitted = (c_int * (2 * max(len(portions), 1)))()
        n = rt.checked(self._lib.flint_rt_sched_commit(self._h, rt.ints(flat), len(portions), rt.ints(tokens), len(tokens),
                                                       emitted, len(portions)))
        out = []
        for i in range(n):
            req, token = self._reqs[emitted[2 * i]], emitted[2 * i + 1]
            req.generated.append(token)
            if token == UNREAD:
                req.n_unread += 1
            out.append((req, token))
        self._pull_touched()
        for p in portions:
            self._pull(p.request)
        self._forget_finished()
        return out

    def _forget_finished(self):
        """Let go of requests that ended long ago (their native records are then used again).  A request with
        unread tokens is kept: its values are still to come."""
        if len(self._reqs) > self.keep_ended:
            for h, r in list(self._reqs.items()):
                if r.state in (FINISHED, FAILED) and not r.n_unread:
                    del self._reqs[h]
                    rt.checked(self._lib.flint_rt_sched_forget(self._h, h))

    def resolve(self, req, token) -> bool:
        """The value of the request's oldest unread token.  True: it is the request's next token.  False: it
        is a stop token (the request ends before it; what ran after it is void), or the request has ended
        at an earlier token or was aborted and the value is dropped."""
        if not self._known(req):
            return False
        self._push_stop(req)
        rc = rt.checked(self._lib.flint_rt_sched_resolve(self._h, req._handle, int(token)))
        if rc == 0:
            req.generated[len(req.generated) - req.n_unread] = int(token)
            req.n_unread -= 1
            return True
        if rc == 1:
            del req.generated[len(req.generated) - req.n_unread:]
            req.n_unread = 0
            self._pull_touched()
            self._pull(req)
        return False

    def steady(self) -> bool:
        """Nothing waits, every running request has exactly its next token left to run, and pages for one
        more token of each are free: the next step can be planned before the last one's tokens are read."""
        return bool(self._lib.flint_rt_sched_steady(self._h))

    def _known(self, req) -> bool:
        """False for a request that ended and was forgotten: its native record may belong to another by now."""
        return self._reqs.get(getattr(req, "_handle", None)) is req

    @property
    def records(self) -> int:
        """Native request records in existence (those of forgotten requests are used again)."""
        return self._lib.flint_rt_sched_records(self._h)

    def abort(self, req):
        if not self._known(req):
            return
        if req.n_unread:
            del req.generated[len(req.generated) - req.n_unread:]
            req.n_unread = 0
        rt.checked(self._lib.flint_rt_sched_abort(self._h, req._handle))
        self._pull_touched()
        self._pull(req)
