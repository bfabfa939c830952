"""The generation engine and the Python entry point.

``Engine`` has the reference engine's interface: ``create`` a session from a prompt,
``step`` the batch, ``poll`` new pieces, ask whether a session is ``finished``, read its
``stats`` and ``close`` it (crates/thuban_generate/src/engine.rs:77-339).  Unlike the reference,
which waits for every step's tokens before it builds the next batch, steady decoding runs one
step ahead: the next step is enqueued with its tokens taken on the device from the sampler's
output, and the host reads a step's tokens while the following step runs.  The stop set is
the model's end-of-sequence ids plus the engine's and the request's extras
(:130-135); the seed of a session is the engine's seed incremented per ``create``
(:129,142).  ``generate`` is the one-call form: token ids (or text, if the model folder
has a ``tokenizer.json``) in, token ids (and text) out.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from pathlib import Path

import torch

from ..errors import ModelError
from ..sampling.params import SamplingParams, SplitMix64
from ..sampling.sampler import BatchSampler
from .model import Model, load_model
from .scheduler import FAILED, FINISHED, UNREAD, Request, Scheduler
from .step import StepEntry


@dataclass
class Piece:
    token: int
    text: str = ""


@dataclass
class GenStats:
    prefill_tokens: int = 0
    decode_tokens: int = 0
    prefill_secs: float = 0.0
    decode_secs: float = 0.0
    preemptions: int = 0


@dataclass
class _Session:
    request: Request
    queue: list = field(default_factory=list)
    created: float = 0.0
    first_token_at: float | None = None
    finished_at: float | None = None


@dataclass
class _Flight:
    """A step that has been enqueued and committed, whose tokens the host has not read yet."""
    portions: list
    ticket: int                # the sampler's
    rows: list                 # the request of each sampled row, in order
    n_tokens: int
    plain: bool                # no row's sampling needs earlier token values on the host (a repeat penalty does)


def load_tokenizer(model_dir):
    """``tokenizer.json`` of the model folder through the ``tokenizers`` package, if both exist."""
    path = Path(model_dir) / "tokenizer.json"
    if not path.is_file():
        return None
    try:
        from tokenizers import Tokenizer
    except ImportError:
        return None
    return Tokenizer.from_file(str(path))


def render_chat(system: str, user: str, history=()) -> str:
    """Phi chat format: ``<|role|>content<|end|>`` per non-empty turn, ending with
    ``<|assistant|>`` (crates/thuban_architectures/src/chat.rs:205-227,258-263)."""
    out = []

    def turn(role, content):
        if content:
            out.append(f"<|{role}|>{content}<|end|>")
    turn("system", system)
    for u, a in history:
        turn("user", u)
        turn("assistant", a)
    turn("user", user)
    out.append("<|assistant|>")
    return "".join(out)


class Engine:
    def __init__(self, model: Model, sampling: SamplingParams | None = None, seed: int = 42, stop=(),
                 tokenizer=None, prefill_chunk: int = 2048, max_step_tokens: int | None = None,
                 run_ahead: bool | None = None):
        self.model = model
        self.sampling = sampling or SamplingParams()
        self.seed = int(seed)
        self.stop = tuple(stop)
        self.tokenizer = tokenizer
        self.scheduler = Scheduler(model.cache,
                                   max_step_tokens=min(max_step_tokens or model.max_step_tokens, model.max_step_tokens),
                                   prefill_chunk=prefill_chunk)
        self.sampler = BatchSampler(model.ops, model.device, max_rows=model.cache.max_slots)
        self.sessions: dict[int, _Session] = {}
        self._next_id = 0
        self.steps = 0
        # steady decoding enqueues the next step before it reads the last one's tokens, if the sampler leaves
        # them where the model can take them
        can = self.sampler.feeds_next_step and model.fed_from is not None
        if run_ahead and not can:
            raise ModelError("running ahead needs a kernel set that keeps the sampled tokens on the device")
        self.run_ahead = can if run_ahead is None else bool(run_ahead)
        self._flight: _Flight | None = None
        self.steps_ahead = 0        # steps that were enqueued before the tokens of the step before were read

    # ------------------------------------------------------------------ sessions
    def create(self, prompt, max_tokens: int, sampling: SamplingParams | None = None, stop_extra=()) -> int:
        """``prompt``: a list of token ids, or text if the engine has a tokenizer."""
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ModelError("a text prompt needs a tokenizer (tokenizer.json in the model folder)")
            prompt = self.tokenizer.encode(prompt).ids
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ModelError("empty prompt")
        for t in prompt:
            if not 0 <= t < self.model.vocab_size:
                raise ModelError(f"token id {t} is outside the vocabulary of {self.model.vocab_size}")
        self.seed = (self.seed + 1) & ((1 << 64) - 1)
        stop = tuple(dict.fromkeys((*self.model.eos_token_ids, *self.stop, *stop_extra)))
        sid = self._next_id
        self._next_id += 1
        req = Request(id=sid, prompt=prompt, max_tokens=int(max_tokens), sampling=sampling or self.sampling,
                      stop=stop, rng=SplitMix64(self.seed), arrival=sid)
        self.sessions[sid] = _Session(req, created=time.perf_counter())
        self.scheduler.add(req)
        if req.state == FAILED:
            raise ModelError(req.error)
        return sid

    def step(self):
        """One batch through the model; returns the number of tokens it ran.  While every running request is
        decoding (and none waits, pages are plentiful, no repeat penalty is set) the step's tokens are read
        during the next call, after that call's batch has been enqueued: they reach ``poll`` one call later.
        A call that finds nothing left to run only brings in the tokens that are still on their way."""
        flight = self._flight
        if flight is not None and not self._may_run_ahead(flight):
            self._land(flight)
            flight = None
        portions = self.scheduler.plan()
        if not portions:
            return self._land(flight) if flight is not None else 0
        place = {id(req): i for i, req in enumerate(flight.rows)} if flight is not None else {}
        entries = []
        for p in portions:
            req, feed = p.request, -1
            if req.n_unread:
                # the request's last token is still on the device: the step takes it from the sampler's output
                if req.n_unread != 1 or p.n_tokens != 1 or p.start != req.n_tokens - 1 or id(req) not in place:
                    raise ModelError("a portion needs token values that the host has not read")
                tokens, feed = [0], place[id(req)]
            else:
                tokens = req.span(p.start, p.n_tokens)
            entries.append(StepEntry(req.slot, p.start, tokens, [p.n_tokens - 1] if p.wants_logits else [], feed))
        logits = self.model.step(entries)
        sampled = [p.request for p in portions if p.wants_logits]
        ticket = self.sampler.launch(logits, [(r.sampling, r.rng, r.generated) for r in sampled])
        plain = all(r.sampling.repeat_penalty == 1.0 or r.sampling.repeat_last_n <= 0 for r in sampled)
        launched = _Flight(portions, ticket, sampled, sum(p.n_tokens for p in portions), plain)
        # everything but the stop set is decided without the tokens' values
        self.scheduler.commit(portions, [UNREAD] * len(sampled))
        self._flight = launched
        self.steps += 1
        if flight is not None:
            self.steps_ahead += 1
            self._land(flight)
        if self._flight is launched and not self._may_run_ahead(launched):
            self._land(launched)
        return launched.n_tokens

    def _may_run_ahead(self, flight) -> bool:
        return self.run_ahead and flight.plain and self.scheduler.steady()

    def _land(self, flight) -> int:
        """Read a flight's tokens (waiting for them) and hand them to their sessions."""
        tokens = self.sampler.read(flight.ticket)
        if any(self.sampler.last_flags):        # a kernel gave up or met a missing page: do not go on with garbage
            self._void_flights(flight)
            self.model.check_status(self.sampler.last_flags)
        now = time.perf_counter()
        for req, tok in zip(flight.rows, tokens):
            if not self.scheduler.resolve(req, tok):
                continue
            s = self.sessions.get(req.id)
            if s is None:
                continue
            if s.first_token_at is None:
                s.first_token_at = now
            text = self.tokenizer.decode([tok]) if self.tokenizer is not None else ""
            s.queue.append(Piece(tok, text))
        for p in flight.portions:
            s = self.sessions.get(p.request.id)
            if s is not None and p.request.state in (FINISHED, FAILED) and s.finished_at is None:
                s.finished_at = now
        if self._flight is flight:
            self._flight = None
        return flight.n_tokens

    def _void_flights(self, flight):
        """After a kernel error: what is in flight is garbage; the requests that wait for it end."""
        for f in (flight, self._flight):
            for req in (f.rows if f is not None else ()):
                if req.n_unread:
                    self.scheduler.abort(req)
        self._flight = None

    def poll(self, sid: int):
        s = self.sessions.get(sid)
        if s is None:
            return []
        out, s.queue = s.queue, []
        return out

    def finished(self, sid: int) -> bool:
        s = self.sessions.get(sid)
        return s is None or (s.request.state in (FINISHED, FAILED) and not s.queue and not s.request.n_unread)

    def error(self, sid: int):
        s = self.sessions.get(sid)
        return s.request.error if s else None

    def stats(self, sid: int):
        s = self.sessions.get(sid)
        if s is None:
            return None
        r = s.request
        end = s.finished_at or time.perf_counter()
        first = s.first_token_at or end
        return GenStats(r.prefill_tokens, r.decode_tokens, first - s.created, end - first, r.preemptions)

    def close(self, sid: int):
        s = self.sessions.pop(sid, None)
        if s is not None and s.request.state not in (FINISHED, FAILED):
            self.scheduler.abort(s.request)

    def has_work(self):
        return self.scheduler.has_work() or self._flight is not None

    # ------------------------------------------------------------------ one call
    def generate(self, prompts, max_tokens: int = 64, sampling: SamplingParams | None = None, stop_extra=()):
        """Run prompts to completion.  Returns one list of generated token ids per prompt."""
        ids = [self.create(p, max_tokens, sampling, stop_extra) for p in prompts]
        out = {i: [] for i in ids}
        while self.has_work():
            if self.step() == 0 and self.has_work():
                raise ModelError("the scheduler made no progress")
            for i in ids:
                out[i].extend(piece.token for piece in self.poll(i))
        for i in ids:
            err = self.error(i)
            self.close(i)
            if err:
                raise ModelError(err)
        return [out[i] for i in ids]


def generate(model_dir, prompts, *, max_tokens=64, temperature=0.7, top_k=20, top_p=0.8, min_p=0.0,
             repeat_penalty=1.0, repeat_last_n=64, seed=42, stop_ids=(), dtype="bfloat16", ctx_size=4096,
             max_requests=8, device="cuda:0", page_size=64, prefill_chunk=2048):
    """Load the model of ``model_dir`` and generate for each prompt (lists of token ids,
    or strings if the folder has a tokenizer).  Option names and defaults are the
    reference's (sampler.rs:24-35; ``--max-tokens``, ``--ctx-size`` of examples/chat/main.rs:14-26)."""
    model = load_model(model_dir, dtype=dtype, device=device, page_size=page_size, max_slots=max_requests,
                       max_context=None if ctx_size is None else min(ctx_size, _max_positions(model_dir)),
                       max_step_tokens=max(prefill_chunk, 64) + max_requests)
    engine = Engine(model, SamplingParams(temperature, top_k, top_p, min_p, repeat_penalty, repeat_last_n), seed,
                    stop_ids, tokenizer=load_tokenizer(model_dir), prefill_chunk=prefill_chunk)
    return engine.generate(prompts, max_tokens)


def _max_positions(model_dir):
    from .model import architecture_of, read_config
    cfg = read_config(model_dir)
    arch = architecture_of(cfg)
    return arch.model_spec(arch.parse_config(cfg)).max_positions
