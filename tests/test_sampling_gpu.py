"""The sampling kernel beside the host sampler with the reference's order of operations."""
import numpy as np
import pytest
import torch

from plain_phimoe import PlainSampler

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run_kernel(ops, logits, params_rows, contexts):
    R, V = logits.shape
    C = max(1, max(len(c) for c in contexts))
    ctx = torch.full((R, C), -1, dtype=torch.int32)
    prm = torch.zeros(R, 8)
    for i, (p, c) in enumerate(zip(params_rows, contexts)):
        ctx[i, :len(c)] = torch.tensor(c, dtype=torch.int32) if c else ctx[i, :0]
        prm[i] = torch.tensor([p["t"], p["k"], p["p"], p["min_p"], p["pen"], p["u"], len(c), 0.0])
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    work = torch.empty(R, V, device=DEV)
    ops.sample(logits.to(DEV), prm.to(DEV), ctx.to(DEV), work, out)
    return out.cpu().tolist(), work.cpu()


def plain_choice(logits, p, context):
    s = PlainSampler(p["t"], p["k"], p["p"], p["min_p"], p["pen"], repeat_last_n=64)
    tok, pr = s.probs(logits.numpy(), context)
    if tok is not None:
        return tok, None, None
    cdf = np.cumsum(pr.astype(np.float64))
    choice = int(np.searchsorted(cdf, p["u"], side="left"))
    margin = float(np.min(np.abs(cdf - p["u"])))
    return min(choice, len(pr) - 1), pr, margin


@pytest.mark.parametrize("V", [17, 1000, 32064])
def test_sample_matches_the_host_sampler(V):
    from flint_b200.csrc.ops import get_ops
    ops = get_ops(DEV)
    g = torch.Generator().manual_seed(V)
    base = dict(t=0.8, k=20, p=0.8, min_p=0.0, pen=1.0)
    variants = [base, dict(base, k=0, p=1.0), dict(base, k=5, p=1.0), dict(base, k=0, p=0.5), dict(base, k=0, p=1.0, min_p=0.3),
                dict(base, t=1.5, k=50, p=0.95, min_p=0.02), dict(base, pen=1.7), dict(base, t=0.0), dict(base, t=0.0, pen=3.0)]
    rows, ctxs, logit_rows = [], [], []
    for vi, v in enumerate(variants):
        for ui, u in enumerate((0.03, 0.31, 0.62, 0.97)):
            lg = torch.randn(V, generator=g) * 3
            if vi == 4:
                lg = (lg * 2).round() / 2            # ties in the logits
            rows.append(dict(v, u=u))
            ctxs.append([int(torch.argmax(lg)), 3, int(torch.argmax(lg))] if v["pen"] != 1.0 else [])
            logit_rows.append(lg)
    logits = torch.stack(logit_rows)
    got, work = run_kernel(ops, logits, rows, ctxs)
    checked = 0
    for i, (p, c) in enumerate(zip(rows, ctxs)):
        want, pr, margin = plain_choice(logits[i], p, c)
        if pr is None:
            assert got[i] == want, f"row {i}: greedy gave {got[i]}, host {want}"
            continue
        assert pr[got[i]] > 0, f"row {i}: token {got[i]} is outside the kept set"
        if margin > 1e-4:                              # away from a boundary of the cumulative sum
            assert got[i] == want, f"row {i} {p}: kernel {got[i]}, host {want}"
            checked += 1
    assert checked >= len(rows) // 2


def test_uniform_logits_and_extremes():
    """All logits equal: top-k keeps the first k indices (ties in index order); u near 0 and 1."""
    from flint_b200.csrc.ops import get_ops
    ops = get_ops(DEV)
    V = 100
    logits = torch.zeros(4, V)
    rows = [dict(t=1.0, k=10, p=1.0, min_p=0.0, pen=1.0, u=u) for u in (0.0, 0.05, 0.55, 0.999999)]
    got, _ = run_kernel(ops, logits, rows, [[]] * 4)
    assert got == [0, 0, 5, 9]
    rows = [dict(t=1.0, k=0, p=0.25, min_p=0.0, pen=1.0, u=u) for u in (0.01, 0.5, 0.99, 0.999999)]
    got, _ = run_kernel(ops, logits, rows, [[]] * 4)
    assert got == [0, 12, 24, 24]                      # the smallest prefix reaching 0.25 is 25 tokens


def test_repeat_penalty_over_more_than_64_tokens():
    """``repeat_last_n`` beyond the width the sampler's buffers start with: the penalty reaches back as far as
    the request says (the buffers grow), as the reference's does for any ``last_n``."""
    from flint_b200.csrc.ops import get_ops
    from flint_b200.sampling.params import SamplingParams, SplitMix64
    from flint_b200.sampling.sampler import BatchSampler
    ops = get_ops(DEV)
    V = 300
    sampler = BatchSampler(ops, DEV, max_rows=2)
    logits = torch.zeros(2, V)
    logits[:, 7] = 5.0            # the favourite, generated 150 tokens ago
    logits[:, 9] = 4.0
    generated = [7] + [11 + (i % 50) for i in range(149)]
    far = SamplingParams(temperature=0.0, repeat_penalty=2.0, repeat_last_n=200)     # sees token 7: 5 / 2 < 4
    near = SamplingParams(temperature=0.0, repeat_penalty=2.0, repeat_last_n=64)     # does not
    got = sampler.sample(logits.to(DEV), [(far, SplitMix64(1), generated), (near, SplitMix64(2), generated)])
    assert got == [9, 7] and sampler.max_context >= 150
    want = [PlainSampler(0.0, 0, 1.0, 0.0, 2.0, repeat_last_n=n).sample(logits[0].numpy(), generated) for n in (200, 64)]
    assert got == want
