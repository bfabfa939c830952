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
    """Runs the trace; returns {step: logits}, the replayer, and the engine's routing
    {(rid, pos): [(i1, i2, g1, g2) per layer]}."""
    rp = Replayer(folder, dtype=dtype, max_tokens=traces.max_tokens_needed(steps), page_size=page_size, **model_kw)
    out, routing, done = {}, {}, {}
    for s in steps:
        rec = {}
        lg = rp.run_step(s["entries"], s["end"], record=rec)
        if lg is not None:
            out[s["step"]] = lg
        ids = [t.cpu() for t in rec.get("experts", [])]
        gates = [t.cpu() for t in rec.get("gates", [])]
        row = 0
        for e in s["entries"]:
            base = done.get(e["id"], 0)
            for j in range(len(e["tokens"])):
                routing[(e["id"], base + j)] = [(int(i[row, 0]), int(i[row, 1]), float(g[row, 0]), float(g[row, 1]))
                                                for i, g in zip(ids, gates)]
                row += 1
            done[e["id"]] = base + len(e["tokens"])
    rp.model.cache.check()
    assert all(g.pages.pool.used_pages == 0 for g in rp.model.cache.groups)
    rp.routing = routing
    return out, rp


def plain_following(folder, reqs, plain, routing, dtype, keep=None, loaded=None):
    """The plain logits with the engine's routing forced where it differs.  Every difference must be
    a near-tie by the plain implementation's own margins (computed on the forced run, so that the
    check is consistent position by position).  Requests without a difference keep their logits."""
    cfg = w = None
    out = dict(plain)
    n_forced = 0
    for rid, toks in reqs.items():
        n = len(toks)
        if any((rid, p) not in routing for p in range(n)):
            continue
        L = len(plain.routing[rid])
        differs = any(routing[(rid, p)][l][:2] != plain.routing[rid][l][p][:2]
                      or abs(routing[(rid, p)][l][2] - plain.routing[rid][l][p][2]) > 2e-2
                      or abs(routing[(rid, p)][l][3] - plain.routing[rid][l][p][3]) > 2e-2
                      for p in range(n) for l in range(L))
        if not differs:
            continue
        assert dtype != "float32", f"{rid}: the 32-bit engine routed differently from the plain implementation"
        if cfg is None:
            cfg, w = loaded or plain_phimoe.load_model_dir(folder)
        forced = [[routing[(rid, p)][l] for p in range(n)] for l in range(L)]
        rec = []
        out[rid] = plain_logits(cfg, w, toks, rec, forced, keep[rid] if keep is not None else None)
        for l in range(L):
            for p in range(n):
                if rec[l][p][5]:
                    n_forced += 1
                    assert rec[l][p][4] < FRAGILE[dtype], (
                        f"{rid} position {p} layer {l}: engine routed {routing[(rid, p)][l]}, plain margin {rec[l][p][4]:.4f}")
    total = sum(len(t) * len(plain.routing[r]) for r, t in reqs.items())
    assert n_forced <= 0.02 * total, f"{n_forced} of {total} routing decisions differ"
    return out


def compare(out, steps, plain, dtype, routing=None, reqs=None, folder=None, keep=None, loaded=None):
    exp_plain = plain_following(folder, reqs, plain, routing, dtype, keep, loaded) if routing is not None else plain
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
