"""The scheduler's decisions with a scripted model (no GPU): admission, portions under a token
budget, decode first, finishing and freeing, and what happens when pages run out."""
import torch

from flint_b200.cache.manager import CacheManager, KVSpec
from flint_b200.engine.scheduler import FAILED, FINISHED, RUNNING, WAITING, Request, Scheduler
from flint_b200.sampling.params import SamplingParams, SplitMix64


def setup(n_pages=16, page=16, slots=4, ctx=256, budget=32, chunk=16, window=0):
    cache = CacheManager({0: KVSpec(1, 16, window)}, {}, page_size=page, n_pages=n_pages, max_slots=slots,
                         max_context=ctx, dtype=torch.float32, device="cpu")
    return cache, Scheduler(cache, max_step_tokens=budget, prefill_chunk=chunk)


def req(i, n_prompt, max_tokens=4, stop=()):
    return Request(id=i, prompt=list(range(1, n_prompt + 1)), max_tokens=max_tokens, sampling=SamplingParams.greedy(),
                   stop=tuple(stop), rng=SplitMix64(i), arrival=i)


def next_token(r):
    """Scripted model: depends only on what the request has run so far."""
    return (len(r.tokens) * 7 + 3) % 97 + 100


def run(sched, reqs, max_steps=500, log=None):
    for r in reqs:
        sched.add(r)
    steps = 0
    while sched.has_work() and steps < max_steps:
        portions = sched.plan()
        if not portions:
            assert not sched.has_work(), "no progress"
            break
        assert sum(p.n_tokens for p in portions) <= sched.max_step_tokens
        assert len({p.request.id for p in portions}) == len(portions)
        if log is not None:
            log.append([(p.request.id, p.start, p.n_tokens, p.wants_logits) for p in portions])
        sched.commit(portions, [next_token(p.request) for p in portions if p.wants_logits])
        sched.cache.check()
        steps += 1
    return steps


def test_prompt_is_cut_into_portions_and_then_decoded():
    cache, s = setup(budget=32, chunk=16)
    r = req(0, 40, max_tokens=3)
    log = []
    run(s, [r], log=log)
    assert [e[0][1:3] for e in log[:3]] == [(0, 16), (16, 16), (32, 8)]
    assert [e[0][3] for e in log[:3]] == [False, False, True]      # logits only where the prompt ends
    assert all(e[0][2] == 1 and e[0][3] for e in log[3:])
    assert r.state == FINISHED and r.finish_reason == "length" and len(r.generated) == 3
    assert (r.prefill_tokens, r.decode_tokens) == (40, 2)
    assert cache.free_slots == 4 and cache.free_pages() == 16     # freed at finish


def test_decodes_go_first_and_the_budget_is_kept():
    cache, s = setup(budget=20, chunk=16)
    a, b = req(0, 5, max_tokens=50), req(1, 60, max_tokens=2)
    log = []
    s.add(a)
    for _ in range(2):
        p = s.plan(); s.commit(p, [next_token(x.request) for x in p if x.wants_logits])
    s.add(b)
    p = s.plan()
    assert [(x.request.id, x.n_tokens) for x in p] == [(0, 1), (1, 16)]   # decode token beside a portion
    s.commit(p, [next_token(x.request) for x in p if x.wants_logits])
    p = s.plan()
    assert [(x.request.id, x.start, x.n_tokens) for x in p] == [(0, 7, 1), (1, 16, 16)]


def test_stop_token_is_not_emitted_and_frees_at_once():
    cache, s = setup()
    r = req(0, 6, max_tokens=10)
    r.stop = (next_token(r),)
    run(s, [r])
    assert r.generated == [] and r.finish_reason == "stop" and cache.free_pages() == 16


def test_waiting_queue_is_first_come_first_served_over_slots():
    cache, s = setup(slots=2, budget=64, chunk=64)
    rs = [req(i, 10, max_tokens=3) for i in range(5)]
    log = []
    run(s, rs, log=log)
    first_seen = {}
    for i, step in enumerate(log):
        for rid, *_ in step:
            first_seen.setdefault(rid, i)
    assert [first_seen[i] for i in range(5)] == sorted(first_seen[i] for i in range(5))
    assert max(len(step) for step in log) <= 2
    assert all(r.state == FINISHED for r in rs)


def test_pages_run_out_the_youngest_is_preempted_and_recomputed():
    cache, s = setup(n_pages=4, page=16, slots=3, budget=64, chunk=64)
    a, b = req(0, 30, max_tokens=20), req(1, 30, max_tokens=20)    # each grows to 50 tokens = 4 pages
    log = []
    run(s, [a, b], log=log)
    assert a.state == b.state == FINISHED
    assert s.preemptions >= 1 and b.preemptions >= 1 and a.preemptions == 0   # the older one is never the victim
    # both produce exactly what they would have produced alone
    for r in (a, b):
        if r.state == FINISHED:
            solo = req(r.id, 30, max_tokens=20)
            c2, s2 = setup(n_pages=16)
            run(s2, [solo])
            assert solo.generated == r.generated
    assert cache.free_pages() == 4 and cache.free_slots == 3


def test_a_request_that_can_never_fit_fails_alone():
    cache, s = setup(n_pages=2, page=16, ctx=256)
    big, small = req(0, 100), req(1, 10, max_tokens=2)
    run(s, [big, small])
    assert big.state == FAILED and "never fit" in big.error
    assert small.state == FINISHED and len(small.generated) == 2
    too_long = req(2, 300)
    s.add(too_long)
    assert too_long.state == FAILED and "context limit" in too_long.error
    empty = req(3, 0)
    s.add(empty)
    assert empty.state == FAILED and "empty" in empty.error


def test_growth_beyond_the_pool_fails_the_lone_request_with_an_error():
    cache, s = setup(n_pages=2, page=16, budget=64, chunk=64)
    r = req(0, 20, max_tokens=100)
    run(s, [r])
    assert r.state == FAILED and "more pages than the pool has" in r.error
    assert len(r.generated) == 13 and cache.free_pages() == 2     # 32 positions held; the 33rd token had no page


def test_window_lets_a_long_request_run_in_few_pages():
    cache, s = setup(n_pages=5, page=16, window=32, budget=16, chunk=16, ctx=256)
    r = req(0, 100, max_tokens=100)
    run(s, [r])
    assert r.state == FINISHED and len(r.generated) == 100 and s.preemptions == 0


def test_context_limit_ends_a_request():
    cache, s = setup(ctx=32)
    r = req(0, 20, max_tokens=100)
    run(s, [r])
    assert r.finish_reason == "context" and len(r.tokens) == 32


def test_random_workloads_keep_every_promise():
    """Random pools, budgets, windows and arrivals (requests join while others run, some are aborted): every
    step keeps the budget and the one-portion-per-request rule, the cache's invariants hold after every
    commit, every request ends (finished, failed alone, or aborted), a finished request produced exactly what
    it produces alone, and in the end every page and slot is free."""
    import random
    for seed in range(12):
        rnd = random.Random(seed)
        page = 16
        n_pages = rnd.randint(3, 24)
        slots = rnd.randint(1, 5)
        window = rnd.choice([0, 0, 32, 48])
        budget = rnd.randint(4, 48)
        chunk = rnd.randint(2, 32)
        cache, s = setup(n_pages=n_pages, page=page, slots=slots, ctx=256, budget=budget, chunk=chunk, window=window)
        todo = [req(i, rnd.randint(1, 90), max_tokens=rnd.randint(1, 40)) for i in range(rnd.randint(3, 10))]
        everyone = list(todo)
        aborted = set()
        steps = 0
        while (todo or s.has_work()) and steps < 5000:
            while todo and (rnd.random() < 0.4 or not s.has_work()):
                s.add(todo.pop(0))
            if rnd.random() < 0.03:
                live = [r for r in everyone if r.state in (WAITING, RUNNING) and r not in todo]
                if live:
                    victim = rnd.choice(live)
                    s.abort(victim)
                    aborted.add(victim.id)
            portions = s.plan()
            assert sum(p.n_tokens for p in portions) <= budget
            assert len({p.request.id for p in portions}) == len(portions)
            for p in portions:
                assert p.n_tokens <= chunk and p.request.state == RUNNING and p.request.slot >= 0
                assert p.start == p.request.n_cached and p.wants_logits == (p.start + p.n_tokens == p.request.n_tokens)
            s.commit(portions, [next_token(p.request) for p in portions if p.wants_logits])
            cache.check()
            steps += 1
        assert steps < 5000, f"seed {seed}: no end"
        for r in everyone:
            assert r.state in (FINISHED, FAILED), (seed, r.id, r.state)
            if r.state == FINISHED and r.id not in aborted:
                solo = req(r.id, len(r.prompt), max_tokens=r.max_tokens)
                _, s2 = setup(n_pages=64, page=page, slots=1, ctx=256, budget=64, chunk=64, window=window)
                run(s2, [solo])
                assert solo.generated == r.generated, (seed, r.id)
            if r.state == FAILED:
                assert r.error
        assert cache.free_pages() == n_pages and cache.free_slots == slots, seed


def test_tokens_committed_unread_are_resolved_later():
    """A step's tokens may be committed before the host knows their values (everything but the stop set is
    decided without them); the values come one step later.  A stop token found then ends the request before
    it and voids what ran after it; the outcome is the one of committing the values at once."""
    from flint_b200.engine.scheduler import UNREAD

    def next_scripted(n_tokens):
        """Scripted model: the token sampled after a request's first n_tokens tokens; 555 is a stop token."""
        return 555 if n_tokens == 9 else 100 + n_tokens

    def drive(ahead):
        cache, s = setup()
        r = req(0, 6, max_tokens=8, stop=(555,))
        q = req(1, 5, max_tokens=2)             # ends by length while its last token is unread
        s.add(r)
        s.add(q)
        pending = None                          # (requests, tokens) of the step whose values are not read yet
        for _ in range(40):
            if not s.has_work():
                break
            if pending and not (ahead and s.steady()):
                for x, t in zip(*pending):
                    s.resolve(x, t)
                pending = None
            portions = s.plan()
            if portions:
                sampled = [p.request for p in portions if p.wants_logits]
                # what the device samples; the host learns it one step later
                values = [next_scripted(x.n_tokens) for x in sampled]
                s.commit(portions, [UNREAD] * len(sampled))
            cache.check()
            if pending:
                for x, t in zip(*pending):
                    s.resolve(x, t)
                pending = None
            if portions:
                pending = (sampled, values)
        if pending:
            for x, t in zip(*pending):
                s.resolve(x, t)
        cache.check()
        assert not s.has_work() and cache.free_slots == 4 and cache.free_pages() == 16
        return r, q

    for ahead in (False, True):
        r, q = drive(ahead)
        assert r.generated == [106, 107, 108] and r.finish_reason == "stop" and r.n_unread == 0, (ahead, r.generated)
        assert q.generated == [105, 106] and q.finish_reason == "length" and q.n_unread == 0
    # a stop token as the last allowed token: the request had ended by length, the reason becomes "stop"
    cache, s = setup()
    r = req(0, 4, max_tokens=1, stop=(7,))
    s.add(r)
    s.commit(s.plan(), [UNREAD])
    assert r.state == FINISHED and r.finish_reason == "length" and r.generated == [UNREAD]
    assert s.resolve(r, 7) is False
    assert r.generated == [] and r.finish_reason == "stop"
    assert s.resolve(r, 9) is False              # nothing unread any more: dropped
    # an aborted request forgets its unread tokens
    r = req(1, 4, max_tokens=5)
    s.add(r)
    s.commit(s.plan(), [UNREAD])
    s.abort(r)
    assert r.generated == [] and s.resolve(r, 3) is False and cache.free_pages() == 16


def test_steady_says_when_the_next_step_needs_no_token_values():
    """Running a step ahead is allowed only while nothing waits, every running request has exactly its next
    token to run, and a page for each of them is free (so that no request can be preempted unread)."""
    from flint_b200.engine.scheduler import UNREAD
    cache, s = setup(n_pages=4, page=16, slots=2, budget=32, chunk=16)
    a, b = req(0, 20, max_tokens=40), req(1, 5, max_tokens=40)
    s.add(a)
    assert not s.steady()                      # a waits
    s.commit(s.plan(), [])                     # first portion of a's prompt: no logits yet
    assert not s.steady()                      # a has prompt left
    s.commit(s.plan(), [UNREAD])
    assert s.steady()                          # a decodes, its token unread, two pages free
    s.add(b)
    assert not s.steady()                      # b waits
    s.resolve(a, 7)
    s.commit(s.plan(), [UNREAD, UNREAD])       # a decodes, b's prompt is run: both now decode with a token unread
    assert a.n_unread == 1 and b.n_unread == 1
    assert cache.free_pages() == 1 and not s.steady()      # two requests, one free page: one of them could be preempted
    s.resolve(a, 8)
    s.resolve(b, 9)
    s.abort(b)
    assert cache.free_pages() == 2 and s.steady()


def test_ended_requests_are_forgotten_and_their_records_used_again():
    """A long-running scheduler does not grow with the number of requests it has served."""
    cache, s = setup(n_pages=16, slots=4, budget=32, chunk=16)
    s.keep_ended = 4
    done = []
    for i in range(60):
        r = req(i, 3 + i % 5, max_tokens=2)
        run(s, [r])
        assert r.state == FINISHED and len(r.generated) == 2
        done.append(r)
    assert s.records <= 8
    s.abort(done[0])                       # a forgotten request: nothing happens, least of all to its record's new owner
    assert s.resolve(done[0], 5) is False
    live = req(100, 4, max_tokens=3)
    s.add(live)
    s.abort(done[1])
    run(s, [])
    assert live.state == FINISHED and len(live.generated) == 3
    assert cache.free_slots == 4 and cache.free_pages() == 16


def test_a_request_preempted_and_admitted_again_in_one_plan_starts_from_zeroed_state():
    """With two pages, the older request's next page costs the younger one its place; the same plan then
    admits the younger one again, into the slot it just gave back.  Its fixed-size state must start from
    zero all the same (a scripted mixer marks the state of every request that ran)."""
    from flint_b200.cache.manager import StateSpec
    cache = CacheManager({0: KVSpec(1, 16, 0)}, {0: StateSpec((4,))}, page_size=16, n_pages=2, max_slots=2,
                         max_context=256, dtype=torch.float32, device="cpu")
    s = Scheduler(cache, max_step_tokens=24, prefill_chunk=8)
    a, b = req(0, 10, 12), req(1, 16, 6)
    s.add(a)
    s.add(b)
    same_slot_again = 0
    for _ in range(300):
        if not s.has_work():
            break
        before = {r.id: (r.slot, r.preemptions) for r in (a, b)}
        portions = s.plan()
        for p in portions:
            r = p.request
            if p.start == 0:
                assert float(cache.state[0][r.slot].abs().sum()) == 0.0, "a request starts on another run's state"
                if r.preemptions > before[r.id][1] and r.slot == before[r.id][0]:
                    same_slot_again += 1
            cache.state[0][r.slot] += 1.0                  # the scripted mixer's running state
        s.commit(portions, [next_token(p.request) for p in portions if p.wants_logits])
        cache.check()
    assert same_slot_again > 0, "the scenario did not come about"
    assert a.state == FINISHED and b.state == FINISHED
