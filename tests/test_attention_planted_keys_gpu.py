"""The bfloat16 attention kernels that serving uses (decode: the TMA-fed kernel with a fixed cut of the key range
and the one that cuts the keys of all rows into equal runs; prefill: the tcgen05 kernel) with one key planted
so that its score stands out.  Random keys among hundreds hide a dropped key or a window that is off by one
(the output moves by about 1/n); a planted key does not: the output of its query head is that key's value, or,
one position outside the window, it is not."""
import math

import pytest
import torch

from flint_b200.cache.manager import CacheView, KVSpec
from kernel_refs import RefOps

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
P = 64


@pytest.fixture(scope="module")
def ops():
    from flint_b200.csrc.ops import get_ops
    return get_ops(DEV)


def close(a, b, tol):
    err = (a.double().cpu() - b.double().cpu()).abs()
    assert (err <= tol + tol * b.double().cpu().abs()).all(), f"max error {err.max().item():.3e}"


def build_rows(cases, nq, nkv, hd, seed):
    """One request per case (length, planted position).  Keys are small random numbers; the planted key is a
    large multiple of the row's query for head 0, so its score is far above every other."""
    g = torch.Generator().manual_seed(seed)
    need = [-(-n // P) for n, _ in cases]
    n_pages = sum(need) + 2
    k = (torch.randn(n_pages, nkv, P, hd, generator=g) * 0.05).to(torch.bfloat16)
    v = torch.randn(n_pages, nkv, P, hd, generator=g).to(torch.bfloat16)
    bt = torch.full((len(cases), max(need) + 1), -1, dtype=torch.int32)
    perm = torch.randperm(n_pages, generator=g).to(torch.int32)
    q = (torch.randn(len(cases), nq * hd, generator=g) * 0.05).to(torch.bfloat16)
    planted = []
    o = 0
    for i, (n, far) in enumerate(cases):
        bt[i, :need[i]] = perm[o:o + need[i]]
        o += need[i]
        page = int(bt[i, far // P])
        k[page, 0, far % P] = (q[i, :hd].float() * 4000.0).to(torch.bfloat16)
        planted.append(v[page, 0, far % P].clone())
    pos = torch.tensor([n - 1 for n, _ in cases], dtype=torch.int32)
    slot = torch.arange(len(cases), dtype=torch.int32)
    return q, k, v, bt, pos, slot, torch.stack(planted)


DECODE_KERNELS = [("stream", None, True), ("tma", (128, 8), True), ("tma", (128, 8), False), ("tma", (64, 13), False),
                  ("tma", (1024, 1), True)]


@pytest.mark.parametrize("kernel,splits,merge", DECODE_KERNELS)
@pytest.mark.parametrize("nq,nkv,hd", [(8, 2, 128), (6, 2, 64)])
def test_decode_finds_a_planted_key_wherever_it_lies(ops, kernel, splits, merge, nq, nkv, hd):
    """The first key, the last and first slot of a page, the edges of a split, the row's own (newest) key."""
    L = 800
    spots = [0, 1, 15, 16, 17, 63, 64, 65, 127, 128, 129, 255, 256, 383, 384, 399, 400, 401, 511, 512, 703, 704,
             L - 2, L - 1]
    cases = [(L, far) for far in spots] + [(n, far) for n, far in ((1, 0), (2, 0), (2, 1), (65, 63), (65, 64), (130, 129))]
    q, k, v, bt, pos, slot, planted = build_rows(cases, nq, nkv, hd, seed=nq + hd)
    spec = KVSpec(nkv, hd, 0)
    dv = CacheView(k.to(DEV), v.to(DEV), bt.to(DEV), P, spec)
    scale = 1 / math.sqrt(hd)
    out = torch.full((len(cases), nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.paged_attention(q.to(DEV), dv, pos.to(DEV), slot.to(DEV), out, nq, nkv, hd, 0, scale, L, kernel=kernel,
                        splits=splits, merge_in_kernel=merge)
    assert int(ops.tc_error.item()) == 0
    exp = torch.zeros(len(cases), nq * hd, dtype=torch.float64)
    RefOps(torch.float64).paged_attention(q, CacheView(k, v, bt, P, spec), pos, slot, exp, nq, nkv, hd, 0, scale, L)
    close(out, exp, 2e-2)
    close(out[:, :hd], planted, 1e-2)              # head 0 returns the planted key's value, and nothing else


@pytest.mark.parametrize("kernel,splits,merge", DECODE_KERNELS[:4])
@pytest.mark.parametrize("window", [40, 100, 257])
def test_decode_window_edge_is_exact(ops, kernel, splits, merge, window):
    """A planted key at distance window - 1 behind the row is its first visible key; at distance window it is
    gone.  Both for keys at the start and the end of a page and in the middle."""
    nq, nkv, hd = 8, 2, 128
    cases, visible = [], []
    for far in (0, 5, 63, 64, 100, 191, 192, 300):
        for dist, seen in ((window - 1, True), (window, False)):
            cases.append((far + dist + 1, far))
            visible.append(seen)
    q, k, v, bt, pos, slot, planted = build_rows(cases, nq, nkv, hd, seed=window)
    spec = KVSpec(nkv, hd, window)
    dv = CacheView(k.to(DEV), v.to(DEV), bt.to(DEV), P, spec)
    scale = 1 / math.sqrt(hd)
    L = max(n for n, _ in cases)
    out = torch.full((len(cases), nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    if splits is not None:
        splits = (splits[0], -(-min(L, window) // splits[0]))
    ops.paged_attention(q.to(DEV), dv, pos.to(DEV), slot.to(DEV), out, nq, nkv, hd, window, scale, L, kernel=kernel,
                        splits=splits, merge_in_kernel=merge)
    assert int(ops.tc_error.item()) == 0
    exp = torch.zeros(len(cases), nq * hd, dtype=torch.float64)
    RefOps(torch.float64).paged_attention(q, CacheView(k, v, bt, P, spec), pos, slot, exp, nq, nkv, hd, window, scale, L)
    close(out, exp, 2e-2)
    for i, seen in enumerate(visible):
        is_planted = torch.allclose(out[i, :hd].float().cpu(), planted[i].float(), atol=2e-2, rtol=1e-2)
        assert is_planted == seen, f"case {cases[i]} window {window}: planted key {'missing' if seen else 'seen'}"


@pytest.mark.parametrize("window", [0, 64, 100, 200])
def test_prefill_on_tensor_cores_finds_planted_keys_and_keeps_the_window_edge(ops, window):
    """A portion of 300 rows that starts 200 tokens deep in its request.  For some rows, two neighbouring rows
    share one query, and a key is planted for it: with a window, at the first position the earlier row still
    sees, which the later row has just lost; without one, at position 0, at a page's last slot, at the row's
    own position.  Tiles of 128 rows by 64 keys: the rows and keys sit on both sides of tile edges."""
    nq, nkv, hd = 8, 2, 128
    start, n_rows = 200, 300
    total = start + n_rows
    g = torch.Generator().manual_seed(window + 3)
    n_pages = -(-total // P) + 2
    k = (torch.randn(n_pages, nkv, P, hd, generator=g) * 0.05).to(torch.bfloat16)
    v = torch.randn(n_pages, nkv, P, hd, generator=g).to(torch.bfloat16)
    bt = torch.full((1, n_pages), -1, dtype=torch.int32)
    bt[0, :n_pages - 2] = torch.randperm(n_pages, generator=g)[:n_pages - 2].to(torch.int32)
    q = (torch.randn(n_rows, nq * hd, generator=g) * 0.05).to(torch.bfloat16)
    checks = []                       # (row, planted position, seen)
    if window:
        for p in (start, 255, 319, 327, 383, 450, total - 2):     # never two neighbours: each planted key has one row
            far = p + 1 - window      # the first key that position p sees
            if far < 0 or p + 1 >= total:
                continue
            r = p - start
            q[r + 1] = q[r]
            checks += [(r, far, True), (r + 1, far, False)]
    else:
        for r, far in ((0, 0), (1, 63), (5, 64), (60, 199), (127, 200 + 127), (128, 200 + 128), (129, 127), (255, 256),
                       (256, 383), (299, total - 1), (298, 1)):
            checks.append((r, far, True))
    used = set()
    planted = {}
    for r, far, seen in checks:
        if (far in used) or not seen:
            continue
        used.add(far)
        page = int(bt[0, far // P])
        k[page, 0, far % P] = (q[r, :hd].float() * 4000.0).to(torch.bfloat16)
        planted[far] = v[page, 0, far % P].clone()
    pos = torch.arange(start, total, dtype=torch.int32)
    slot = torch.zeros(n_rows, dtype=torch.int32)
    tiles = []
    for r in range(0, n_rows, 128):
        tiles += [r, min(128, n_rows - r), 0, start + r]
    spec = KVSpec(nkv, hd, window)
    dv = CacheView(k.to(DEV), v.to(DEV), bt.to(DEV), P, spec)
    scale = 1 / math.sqrt(hd)
    out = torch.full((n_rows, nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.attention_prefill_tc(q.to(DEV), dv, torch.tensor(tiles, dtype=torch.int32, device=DEV), len(tiles) // 4, out, nq,
                             nkv, hd, window, scale)
    assert int(ops.tc_error.item()) == 0
    exp = torch.zeros(n_rows, nq * hd, dtype=torch.float64)
    RefOps(torch.float64).paged_attention(q, CacheView(k, v, bt, P, spec), pos, slot, exp, nq, nkv, hd, window, scale, total)
    close(out, exp, 2e-2)
    for r, far, seen in checks:
        if far not in planted:
            continue
        is_planted = torch.allclose(out[r, :hd].float().cpu(), planted[far].float(), atol=2e-2, rtol=1e-2)
        # a row may see a key planted for another row as well; what is checked is the row the key was planted for,
        # and its neighbour with the same query one position later
        assert is_planted == seen, f"row {r} (position {start + r}), key {far}, window {window}"


@pytest.mark.parametrize("kernel", ["stream", "tma"])
@pytest.mark.parametrize("window,far", [(0, 5), (0, 70000), (100000, 131072 - 100000), (100000, 131072 - 100001)])
def test_decode_over_131072_keys(ops, kernel, window, far):
    """One row at the end of the longest context the model allows, over scattered pages: against float64, and
    with a planted key far back that must be found (or, one position outside a window of 100,000, must not)."""
    nq, nkv, hd, L = 8, 2, 128, 131072
    q, k, v, bt, pos, slot, planted = build_rows([(L, far)], nq, nkv, hd, seed=far % 97)
    spec = KVSpec(nkv, hd, window)
    dv = CacheView(k.to(DEV), v.to(DEV), bt.to(DEV), P, spec)
    scale = 1 / math.sqrt(hd)
    out = torch.full((1, nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.paged_attention(q.to(DEV), dv, pos.to(DEV), slot.to(DEV), out, nq, nkv, hd, window, scale, L, kernel=kernel)
    assert int(ops.tc_error.item()) == 0
    exp = torch.zeros(1, nq * hd, dtype=torch.float64)
    RefOps(torch.float64).paged_attention(q, CacheView(k, v, bt, P, spec), pos, slot, exp, nq, nkv, hd, window, scale, L)
    close(out, exp, 2e-2)
    seen = window == 0 or far >= L - window
    assert torch.allclose(out[0, :hd].float().cpu(), planted[0].float(), atol=2e-2, rtol=1e-2) == seen
