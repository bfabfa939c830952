"""Shared helpers of the GPU engine tests: the plain implementation's logits and routing for a set of
requests, the replay of a trace with the engine's routing recorded, and the comparison of the two."""
import torch

import plain_phimoe
import traces
from flint_b200.engine.replay import Replayer

# float32: the engine's float32 kernels against float64 arithmetic.  bfloat16: activations are rounded
# to 8 bits of mantissa between kernels (2^-9 relative each); weights are the same bfloat16 values on
# both sides.  Sparsemixer routing is discontinuous (an arg-max and a mask threshold), so rounding can
# flip a decision whose margin is within the rounding noise, and the logits after such a flip are not
# comparable with an unflipped run.  The tests therefore compare routing first: a difference is accepted
# only where the plain implementation itself says that the decision was a near-tie (FRAGILE); the plain
# implementation is then run again following the engine at exactly those decisions, and every logit at
# every position is compared.
TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}
FRAGILE = {"float32": 1e-5, "bfloat16": 1e-2}     # as a fraction of the row's largest router logit


class Plain(dict):
    """request id -> logits [len, vocab]; ``.routing[rid][layer][pos]`` = (i1, i2, g1, g2, fragility)."""
    routing = None


class RowsAt:
    """Logits of a few positions of a request, indexed by position like a [len, vocab] tensor."""

    def __init__(self, positions, logits):
        self.index = {p: i for i, p in enumerate(positions)}
        self.logits = logits

    def __getitem__(self, pos):
        return self.logits[self.index[pos]]

    def abs(self):
        return self.logits.abs()


def plain_logits(cfg, w, tokens, rec, forced=None, positions=None):
    """The plain implementation's logits of one request: everywhere, or at ``positions`` only."""
    if positions is None:
        return plain_phimoe.forward(cfg, w, tokens, rec, forced)
    positions = sorted(positions)
    return RowsAt(positions, plain_phimoe.forward(cfg, w, tokens, rec, forced, logit_rows=positions))


def plain_all(folder, reqs, keep=None, loaded=None):
    """``keep``: request id -> the positions whose logits are computed (default: all)."""
    cfg, w = loaded or plain_phimoe.load_model_dir(folder)
    out = Plain()
    out.routing = {}
    for rid, t in reqs.items():
        rec = []
        out[rid] = plain_logits(cfg, w, t, rec, positions=keep[rid] if keep is not None else None)
        out.routing[rid] = rec
    return out


def replay(folder, dtype, steps, page_size, **model_kw):
    """Runs the trace; returns {step: logits} and the replayer, which carries the engine's routing
    ``rp.routing[(rid, pos)] = [(i1, i2, g1, g2) per layer]`` and the router logits behind it
    ``rp.router_logits[(rid, pos)] = [tensor [E] per layer]``."""
    rp = Replayer(folder, dtype=dtype, max_tokens=traces.max_tokens_needed(steps), page_size=page_size, **model_kw)
    out, routing, router_logits, done = {}, {}, {}, {}
    for s in steps:
        rec = {}
        lg = rp.run_step(s["entries"], s["end"], record=rec)
        if lg is not None:
            out[s["step"]] = lg
        ids = [t.cpu() for t in rec.get("experts", [])]
        gates = [t.cpu() for t in rec.get("gates", [])]
        logits = [t.cpu() for t in rec.get("router_logits", [])]
        assert len(logits) == len(ids), "the engine did not record the router logits of every layer"
        row = 0
        for e in s["entries"]:
            base = done.get(e["id"], 0)
            for j in range(len(e["tokens"])):
                routing[(e["id"], base + j)] = [(int(i[row, 0]), int(i[row, 1]), float(g[row, 0]), float(g[row, 1]))
                                                for i, g in zip(ids, gates)]
                router_logits[(e["id"], base + j)] = [l[row] for l in logits]
                row += 1
            done[e["id"]] = base + len(e["tokens"])
    rp.model.cache.check()
    assert all(g.pages.pool.used_pages == 0 for g in rp.model.cache.groups)
    rp.routing = routing
    rp.router_logits = router_logits
    return out, rp


def check_selection(cfg, routing, router_logits):
    """The engine's choice of experts and its gates are exactly what the sparsemixer rule gives for the
    engine's own router logits (float32 values; a decision may differ only where those logits sit within
    float32 rounding of a tie or of a mask threshold)."""
    eps = cfg.get("router_jitter_noise", cfg.get("jitter_eps", 0.01))
    for key, per_layer in routing.items():
        for layer, (i1, i2, g1, g2) in enumerate(per_layer):
            s = router_logits[key][layer].double()
            w1, wg1, w2, wg2 = plain_phimoe.sparsemixer_top2(s, eps)
            if (w1, w2) == (i1, i2) and abs(float(wg1) - g1) < 1e-4 and abs(float(wg2) - g2) < 1e-4:
                continue
            assert plain_phimoe.routing_fragility(s, eps) < 1e-6, (
                f"{key} layer {layer}: the engine chose {(i1, i2, g1, g2)} from logits {s.tolist()}, "
                f"the rule gives {(w1, w2, float(wg1), float(wg2))}")


def plain_following(folder, reqs, plain, routing, dtype, keep=None, loaded=None, router_logits=None,
                    max_differing=None):
    """The plain logits with the engine's routing forced where it differs, and the proof that every
    difference is legitimate: (1) the engine's decision is exactly the sparsemixer rule applied to its own
    router logits (``check_selection``), and (2) those logits agree with the plain implementation's (of the
    forced run, position by position) within the tolerance of the final logits, and (3) where a decision
    differs, the plain implementation's own margin at that row (the smallest change of one logit that would
    change its decision) is no larger than what the measured difference between the two rows of logits can
    bridge (two logits moving against each other: twice the largest difference, and a little for the mask
    ratio's denominator).  Requests without a difference keep their logits.
    ``max_differing``: the largest accepted share of differing decisions (default 2 % in bfloat16, 0.05 % in
    32-bit)."""
    cfg, w = loaded or plain_phimoe.load_model_dir(folder)
    if router_logits is not None:
        check_selection(cfg, routing, router_logits)
    out = dict(plain)
    n_forced = 0
    worst_router = 0.0
    for rid, toks in reqs.items():
        n = len(toks)
        if any((rid, p) not in routing for p in range(n)):
            continue
        L = len(plain.routing[rid])
        differs = any(routing[(rid, p)][l][:2] != plain.routing[rid][l][p][:2]
                      or abs(routing[(rid, p)][l][2] - plain.routing[rid][l][p][2]) > 2e-2
                      or abs(routing[(rid, p)][l][3] - plain.routing[rid][l][p][3]) > 2e-2
                      for p in range(n) for l in range(L))
        rec = plain.routing[rid]
        if differs:
            forced = [[routing[(rid, p)][l] for p in range(n)] for l in range(L)]
            rec = []
            out[rid] = plain_logits(cfg, w, toks, rec, forced, keep[rid] if keep is not None else None)
            n_forced += sum(1 for l in range(L) for p in range(n) if rec[l][p][5])
        if router_logits is None:
            # no logits to explain a difference with: the plain implementation's own margin must call it a near-tie
            for l in range(L):
                for p in range(n):
                    assert not rec[l][p][5] or rec[l][p][4] < FRAGILE[dtype], (
                        f"{rid} position {p} layer {l}: engine routed {routing[(rid, p)][l]}, plain margin {rec[l][p][4]:.4f}")
            continue
        for l in range(L):
            want = torch.stack([rec[l][p][6] for p in range(n)])
            got = torch.stack([router_logits[(rid, p)][l] for p in range(n)]).double()
            err = float((got - want).abs().max() / want.abs().max())
            worst_router = max(worst_router, err)
            assert err <= TOL[dtype], f"{rid} layer {l}: router logits differ by {err:.3e} of the largest"
            if differs:
                row_err = (got - want).abs().max(dim=1).values / want.abs().max(dim=1).values
                for p in range(n):
                    assert not rec[l][p][5] or rec[l][p][4] <= 2.5 * float(row_err[p]) + 1e-6, (
                        f"{rid} position {p} layer {l}: engine routed {routing[(rid, p)][l]}; the plain margin "
                        f"{rec[l][p][4]:.5f} is beyond what a logit difference of {float(row_err[p]):.5f} explains")
    total = sum(len(t) * len(plain.routing[r]) for r, t in reqs.items())
    if max_differing is None:
        max_differing = 0.02 if dtype == "bfloat16" else 0.0005
    assert n_forced <= max_differing * total, f"{n_forced} of {total} routing decisions differ"
    return out


def compare(out, steps, plain, dtype, routing=None, reqs=None, folder=None, keep=None, loaded=None,
            router_logits=None, max_differing=None):
    exp_plain = plain_following(folder, reqs, plain, routing, dtype, keep, loaded, router_logits, max_differing) \
        if routing is not None else plain
    exp = traces.expected_rows(steps, exp_plain)
    assert set(out) == set(exp)
    scale = max(float(v.abs().max()) for v in plain.values())
    worst = 0.0
    for k, rows in exp.items():
        want = torch.stack(rows)
        assert out[k].shape == want.shape
        assert torch.isfinite(out[k]).all()
        worst = max(worst, (out[k].double() - want).abs().max().item())
    assert worst <= TOL[dtype] * scale, f"max error {worst:.3e} against a largest logit of {scale:.3f}"
    return worst
