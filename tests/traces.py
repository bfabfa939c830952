"""Traces in the replay tool's format, for the same requests cut in different ways."""
from __future__ import annotations

import random


def make_requests(vocab, lengths, seed=0):
    r = random.Random(seed)
    return {f"r{i}": [r.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}


def _step(i, entries, end=()):
    return {"step": i, "entries": entries, "end": list(end)}


def _wanted(rid, start, places, keep):
    """``places`` (indices into a portion that starts at position ``start``) restricted to the
    positions that ``keep`` (request id -> set of positions, or None for all) names."""
    if keep is None:
        return list(places)
    return [w for w in places if start + w in keep[rid]]


def whole(reqs, keep=None):
    """Each request alone and whole, logits at every place (or at the kept positions)."""
    return [_step(i, [{"id": rid, "tokens": t, "want": _wanted(rid, 0, range(len(t)), keep)}], [rid])
            for i, (rid, t) in enumerate(reqs.items())]


def tail_decoded(reqs, tail=32, keep=None):
    """All but the last ``tail`` tokens in one step, then the rest one token per step."""
    steps = []
    for rid, t in reqs.items():
        head = max(len(t) - tail, 1)
        steps.append(_step(len(steps), [{"id": rid, "tokens": t[:head], "want": _wanted(rid, 0, [head - 1], keep)}]))
        for j in range(head, len(t)):
            steps.append(_step(len(steps), [{"id": rid, "tokens": [t[j]], "want": _wanted(rid, j, [0], keep)}],
                               [rid] if j == len(t) - 1 else []))
        if head == len(t):
            steps[-1]["end"] = [rid]
    return steps


def portions(reqs, sizes=(7, 2, 13, 3, 5, 2, 16, 1, 2, 31, 2, 64), keep=None):
    """Portions of changing size, down to two tokens, logits everywhere."""
    steps = []
    for rid, t in reqs.items():
        i, k = 0, 0
        while i < len(t):
            n = min(sizes[k % len(sizes)], len(t) - i)
            k += 1
            steps.append(_step(len(steps), [{"id": rid, "tokens": t[i:i + n], "want": _wanted(rid, i, range(n), keep)}],
                               [rid] if i + n == len(t) else []))
            i += n
    return steps


def mixed(reqs, seed=0, max_live=4, decode_tail=12, sizes=(2, 2, 3, 5, 8, 16, 33), keep=None):
    """Up to ``max_live`` live requests; each step takes portions of some beside single tokens of
    others; some requests sit a step out; finished requests leave and new ones come in."""
    rnd = random.Random(seed)
    waiting = list(reqs.items())
    live = {}      # rid -> tokens done
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, _ = waiting.pop(0)
            live[rid] = 0
        entries, end = [], []
        for rid in list(live):
            t, done = reqs[rid], live[rid]
            if len(live) > 1 and rnd.random() < 0.15:
                continue                               # left out of this step, goes on later
            left = len(t) - done
            if left <= decode_tail:
                n = 1
            else:
                n = min(rnd.choice(list(sizes)), left - decode_tail)
            want = sorted(set(rnd.sample(range(n), k=min(n, rnd.choice([0, 1, 2, n])))) | ({n - 1} if n == 1 else set()))
            entries.append({"id": rid, "tokens": t[done:done + n], "want": _wanted(rid, done, want, keep)})
            live[rid] = done + n
            if live[rid] == len(t):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append(_step(len(steps), entries, end))
    return steps


def max_tokens_needed(steps, unit=64):
    """The most tokens live requests hold at any time, each rounded up to ``unit``."""
    held, worst = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(-(-n // unit) * unit for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return worst


def expected_rows(steps, plain_logits):
    """For each step with wanted places: the plain implementation's logits rows, in order.
    ``plain_logits``: request id -> tensor [len, vocab]."""
    done, out = {}, {}
    for s in steps:
        rows = []
        for e in s["entries"]:
            base = done.get(e["id"], 0)
            rows += [plain_logits[e["id"]][base + w] for w in e["want"]]
            done[e["id"]] = base + len(e["tokens"])
        if rows:
            out[s["step"]] = rows
    return out
