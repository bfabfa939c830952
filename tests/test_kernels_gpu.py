"""Each CUDA kernel alone beside its plain reference, at sizes other than the engine's."""
import math

import pytest
import torch

from flint_b200.cache.manager import CacheView, KVSpec
from kernel_refs import RefOps

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from flint_b200.csrc.ops import get_ops
    return get_ops(DEV)


@pytest.fixture(scope="module")
def ref():
    return RefOps(torch.float64)


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def close(a, b, rtol, atol):
    a, b = a.double().cpu(), b.double().cpu()
    err = (a - b).abs()
    bound = atol + rtol * b.abs()
    assert (err <= bound).all(), f"max err {err.max().item():.3e}, worst excess {(err - bound).max().item():.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,V", [(1, 40, 17), (37, 1000, 333), (5, 4096, 64)])
def test_embed(ops, ref, dtype, T, H, V):
    table = rnd(V, H, dtype=dtype)
    ids = torch.randint(0, V, (T,), dtype=torch.int32)
    out = torch.empty(T, H, device=DEV)
    ops.embed(ids.to(DEV), table.to(DEV), out, 1.0)
    exp = torch.empty(T, H)
    ref.embed(ids, table, exp)
    assert torch.equal(out.cpu(), exp)


@pytest.mark.parametrize("mode,bias", [("layer", True), ("layer", False), ("rms", False)])
@pytest.mark.parametrize("T,H", [(1, 24), (33, 96), (7, 1000), (3, 4096), (2, 5000)])
def test_norm(ops, ref, mode, bias, T, H):
    x = rnd(T, H, scale=3.0) + 1.5          # a mean far from zero shows a one-pass variance
    gamma, beta = 1 + rnd(H, seed=1) * 0.1, (rnd(H, seed=2) * 0.1 if bias else None)
    o32, o16 = torch.empty(T, H, device=DEV), torch.empty(T, H, device=DEV, dtype=torch.bfloat16)
    ops.norm(x.to(DEV), gamma.to(DEV), beta.to(DEV) if bias else None, 1e-5, mode, out_f32=o32, out_bf16=o16)
    e32 = torch.empty(T, H)
    ref.norm(x, gamma, beta, 1e-5, mode, out_f32=e32)
    close(o32, e32, 1e-5, 1e-5)
    close(o16, e32, 1e-2, 1e-2)
    # gathered rows
    idx = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32)
    o = torch.empty(3, H, device=DEV)
    ops.norm(x.to(DEV), gamma.to(DEV), beta.to(DEV) if bias else None, 1e-5, mode, out_f32=o, row_index=idx.to(DEV))
    close(o, e32[idx.long()], 1e-5, 1e-5)


@pytest.mark.parametrize("T,H,E,wd", [(1, 4096, 16, torch.bfloat16), (9, 96, 6, torch.float32), (33, 64, 4, torch.bfloat16),
                                      (5, 1000, 7, torch.float32), (3, 8192, 16, torch.bfloat16), (2, 2052, 3, torch.float32),
                                      (301, 4096, 16, torch.bfloat16), (258, 96, 6, torch.float32),
                                      (4, 16384, 40, torch.bfloat16), (8, 4096, 64, torch.float32),
                                      (16, 1536, 16, torch.bfloat16), (300, 1000, 7, torch.bfloat16),
                                      (260, 2048, 40, torch.bfloat16), (1030, 4096, 16, torch.bfloat16)])
@pytest.mark.parametrize("mode", ["layer", "rms"])
def test_row_norm_with_pending_additions_and_router(ops, ref, T, H, E, wd, mode):
    """The fused row kernel beside the separate references: split-K partial sums + bias, the gated sum
    of two expert rows, the norm, and the routing of the normalised row.  Up to 16 rows of at least 512
    values are shared by a cluster of blocks each; more rows, or narrower ones, get a block each."""
    from flint_b200.parts.base import Pending, RouterRequest
    x0 = rnd(T, H, scale=2.0) + 0.5
    gamma, beta = 1 + rnd(H, seed=1) * 0.1, (rnd(H, seed=2) * 0.1 if mode == "layer" else None)
    partials, bias = rnd(13 if H == 4096 else 3, T, H, seed=3), rnd(H, seed=4)
    y = rnd(2 * T, H, seed=5)
    row_of = torch.randperm(2 * T, generator=torch.Generator().manual_seed(6)).to(torch.int32).view(T, 2)
    gts = torch.rand(T, 2)
    wr = rnd(E, H, dtype=wd, seed=7, scale=0.05)
    dev = lambda t: t.to(DEV) if t is not None else None
    for use_partials, use_comb, use_router in ((True, False, False), (False, True, True), (True, True, True), (False, False, True)):
        pend_d = Pending(partials=dev(partials) if use_partials else None, bias=dev(bias) if use_partials else None,
                         y=dev(y) if use_comb else None, row_of=dev(row_of) if use_comb else None,
                         gates=dev(gts) if use_comb else None) if (use_partials or use_comb) else None
        pend_r = Pending(partials=partials if use_partials else None, bias=bias if use_partials else None,
                         y=y if use_comb else None, row_of=row_of if use_comb else None,
                         gates=gts if use_comb else None) if (use_partials or use_comb) else None
        xd, xr = x0.clone().to(DEV), x0.clone().double()
        o32, o16 = torch.empty(T, H, device=DEV), torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
        req = RouterRequest(dev(wr), 0.05, torch.empty(T, 2, dtype=torch.int32, device=DEV),
                            torch.empty(T, 2, device=DEV)) if use_router else None
        ops.row_norm(xd, dev(gamma), dev(beta), 1e-5, mode, out_f32=o32, out_bf16=o16, pending=pend_d, router=req)
        e32 = torch.empty(T, H, dtype=torch.float64)
        rreq = RouterRequest(wr, 0.05, torch.empty(T, 2, dtype=torch.int32), torch.empty(T, 2, dtype=torch.float64)) \
            if use_router else None
        RefOps(torch.float64).row_norm(xr, gamma, beta, 1e-5, mode, out_f32=None, pending=pend_r)
        RefOps(torch.float64).norm(xr, gamma, beta, 1e-5, mode, out_f32=e32)
        close(xd, xr, 1e-6, 1e-5)                       # the residual stream was updated in place
        close(o32, e32, 1e-5, 1e-5)
        close(o16, e32, 1e-2, 1e-2)
        if use_router:
            RefOps(torch.float64).router_sparsemixer(e32, wr, 0.05, rreq.expert_ids, rreq.gates)
            assert torch.equal(req.expert_ids.cpu(), rreq.expert_ids)
            close(req.gates, rreq.gates, 1e-4, 1e-5)
    # gathered rows with a pending sum, and the additions alone
    idx = torch.tensor([T - 1, 0], dtype=torch.int32)
    xd, xr = x0.clone().to(DEV), x0.clone().double()
    o = torch.empty(2, H, device=DEV)
    ops.row_norm(xd, dev(gamma), dev(beta), 1e-5, mode, out_f32=o, row_index=idx.to(DEV),
                 pending=Pending(partials=dev(partials), bias=dev(bias)))
    xr += partials.double().sum(0) + bias.double()
    e = torch.empty(T, H, dtype=torch.float64)
    RefOps(torch.float64).norm(xr, gamma, beta, 1e-5, mode, out_f32=e)
    close(o, e[idx.long()], 1e-5, 1e-5)
    xd = x0.clone().to(DEV)
    ops.apply_pending(xd, Pending(y=dev(y), row_of=dev(row_of), gates=dev(gts)))
    xr = x0.clone().double()
    RefOps(torch.float64).moe_combine(xr, y, row_of, gts)
    close(xd, xr, 1e-6, 1e-5)


def test_gemm_partials_and_rope_sum_them(ops, ref):
    """A product left as partial sums over pieces of K, summed by the rotary kernel with the bias."""
    T, nq, nkv, hd, H = 5, 4, 2, 32, 4096
    x, w, b = rnd(T, H, dtype=torch.bfloat16), rnd((nq + 2 * nkv) * hd, H, dtype=torch.bfloat16, seed=1, scale=0.05), rnd((nq + 2 * nkv) * hd, seed=2)
    parts = ops.gemm_partials(x.to(DEV), w.to(DEV))
    assert parts.shape[0] > 1 and parts.shape[1:] == (T, (nq + 2 * nkv) * hd)
    exp = x.double() @ w.double().T
    close(parts.sum(0), exp, 1e-5, 1e-3)
    P = 16
    k, v, bt = make_cache(4, nkv, P, hd, torch.bfloat16, 1, 4)
    bt[0, :2] = torch.tensor([2, 1], dtype=torch.int32)
    dv, cv = views(k, v, bt, P, nkv, hd, 0)
    pos, slot = torch.arange(3, 3 + T, dtype=torch.int32), torch.zeros(T, dtype=torch.int32)
    ang = torch.arange(64, dtype=torch.float64)[:, None] * (10000.0 ** (-torch.arange(hd // 2, dtype=torch.float64) * 2 / hd))
    cos, sin = torch.cos(ang).float(), torch.sin(ang).float()
    q_d = torch.empty(T, nq * hd, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.rope_kv_write(parts, pos.to(DEV), slot.to(DEV), cos.to(DEV), sin.to(DEV), hd, q_d, dv, nq, nkv, hd, True, status,
                      bias=b.to(DEV))
    q_r = torch.empty(T, nq * hd, dtype=torch.float64)
    ref.rope_kv_write(exp + b.double(), pos, slot, cos, sin, hd, q_r, cv, nq, nkv, hd, True, None)
    close(q_d, q_r, 1e-2, 1e-2)
    close(dv.k, cv.k, 1e-2, 1e-2)
    close(dv.v, cv.v, 1e-2, 1e-2)


GEMM_SHAPES = [(1, 16, 64), (3, 17, 33), (64, 64, 64), (65, 130, 100), (200, 96, 80), (7, 384, 96), (130, 250, 1000)]


@pytest.mark.parametrize("xd,wd,od", [(torch.float32,) * 3, (torch.bfloat16, torch.bfloat16, torch.float32),
                                      (torch.bfloat16, torch.bfloat16, torch.bfloat16),
                                      (torch.bfloat16, torch.float32, torch.float32)])
@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_dense(ops, ref, xd, wd, od, M, N, K):
    x, w, b = rnd(M, K, dtype=xd), rnd(N, K, dtype=wd, seed=1), rnd(N, seed=2)
    out0 = rnd(M, N, dtype=od, seed=3)
    for bias, acc in ((None, False), (b, False), (b, True)):
        out = out0.clone().to(DEV)
        ops.gemm(x.to(DEV), w.to(DEV), out, bias=bias.to(DEV) if bias is not None else None, accumulate=acc)
        exp = out0.clone().double()
        ref.gemm(x, w, exp, bias=bias, accumulate=acc)
        tol = (1e-5, 1e-4) if od == torch.float32 else (1e-2, 1e-2)
        close(out, exp, *tol)


def test_gemm_strided_output(ops, ref):
    x, w = rnd(9, 40), rnd(24, 40, seed=1)
    full = torch.zeros(9, 100, device=DEV)
    ops.gemm(x.to(DEV), w.to(DEV), full[:, :24])
    exp = torch.zeros(9, 24, dtype=torch.float64)
    ref.gemm(x, w, exp)
    close(full[:, :24], exp, 1e-5, 1e-4)
    assert (full[:, 24:] == 0).all()


@pytest.mark.parametrize("act", ["silu", "gelu_pytorch_tanh"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("I", [80, 72])          # a multiple of the pairing block of 16, and not
def test_gated_and_grouped(ops, ref, act, dtype, I):
    T, H, E = 75, 96, 6
    ids = torch.randint(0, E, (T, 2), dtype=torch.int32)
    ids[:, 1] = (ids[:, 0] + 1 + ids[:, 1] % (E - 1)) % E
    ids[ids == 4] = 0                      # expert 4 gets no rows
    ids[:, 1] = torch.where(ids[:, 1] == ids[:, 0], (ids[:, 0] + 1) % E, ids[:, 1])
    plan = ops.moe_plan(ids.to(DEV), E, 64)
    rplan = ref.moe_plan(ids, E, 64)
    assert torch.equal(plan.counts.cpu(), rplan.counts) and torch.equal(plan.offsets.cpu(), rplan.offsets)
    assert int(plan.n_tiles.item()) == int(rplan.n_tiles.item())
    nt = int(plan.n_tiles)
    assert torch.equal(plan.tile_expert.cpu()[:nt], rplan.tile_expert[:nt])
    assert torch.equal(plan.tile_row0.cpu()[:nt], rplan.tile_row0[:nt])
    # every (token, choice) has a row of its own inside its expert's range, and token_of inverts row_of
    row_of, token_of = plan.row_of.cpu().long(), plan.token_of.cpu().long()
    assert sorted(row_of.reshape(-1).tolist()) == list(range(2 * T))
    off = plan.offsets.cpu().long()
    e_of = ids.long()
    assert ((row_of >= off[e_of]) & (row_of < off[e_of + 1])).all()
    assert torch.equal(token_of[row_of], torch.arange(T)[:, None].expand(T, 2))

    x = rnd(T, H, dtype=dtype)
    xs = torch.empty(2 * T, H, dtype=dtype, device=DEV)
    ops.gather_rows(x.to(DEV), plan.token_of, xs)
    assert torch.equal(xs.cpu(), x[token_of])
    # plan and gather in one launch (few rows), with ranks by position: the same counts and tiles, a valid order
    for n_tok in (T, 1, 9):
        sub = ids[:n_tok].contiguous()
        rp = ref.moe_plan(sub, E, 64)
        dplan, dxs = ops.moe_dispatch(sub.to(DEV), E, 64, x[:n_tok].to(DEV))
        assert torch.equal(dplan.counts.cpu(), rp.counts) and torch.equal(dplan.offsets.cpu(), rp.offsets)
        nt2 = int(dplan.n_tiles.item())
        assert nt2 == int(rp.n_tiles.item())
        assert torch.equal(dplan.tile_expert.cpu()[:nt2], rp.tile_expert[:nt2])
        assert torch.equal(dplan.tile_row0.cpu()[:nt2], rp.tile_row0[:nt2])
        d_row, d_tok = dplan.row_of.cpu().long(), dplan.token_of.cpu().long()
        assert torch.equal(d_row, rp.row_of.long())            # both rank by position
        assert torch.equal(d_tok[d_row], torch.arange(n_tok)[:, None].expand(n_tok, 2))
        assert torch.equal(dxs.cpu(), x[:n_tok][d_tok])
    w1, w3, w2 = (rnd(E, I, H, dtype=dtype, seed=1, scale=0.1), rnd(E, I, H, dtype=dtype, seed=2, scale=0.1),
                  rnd(E, H, I, dtype=dtype, seed=3, scale=0.1))
    w13 = ops.pair_gate_up(w1, w3).contiguous()        # the kernels' layout; the reference keeps its own
    r13 = ref.pair_gate_up(w1, w3)
    a = torch.empty(2 * T, I, dtype=dtype, device=DEV)
    ops.gated_gemm(xs, w13.to(DEV), a, act, plan)
    # the reference works on the same row order
    from flint_b200.csrc.ops import MoePlan
    cplan = MoePlan(E, 64, plan.max_tiles, *(t.cpu() for t in (plan.counts, plan.offsets, plan.row_of, plan.token_of,
                                                             plan.tile_expert, plan.tile_row0, plan.n_tiles)))
    ea = torch.zeros(2 * T, I, dtype=torch.float64)
    ref.gated_gemm(xs.cpu(), r13, ea, act, cplan)
    tol = (1e-5, 1e-4) if dtype == torch.float32 else (2e-2, 2e-2)
    close(a, ea, *tol)
    y = torch.empty(2 * T, H, device=DEV)
    ops.grouped_gemm(a, w2.to(DEV), y, plan)
    ey = torch.zeros(2 * T, H, dtype=torch.float64)
    ref.grouped_gemm(a.cpu(), w2, ey, cplan)
    close(y, ey, 1e-5, 1e-5)
    gates = torch.rand(T, 2)
    h0 = rnd(T, H, seed=9)
    h = h0.clone().to(DEV)
    ops.moe_combine(h, y, plan.row_of, gates.to(DEV))
    eh = h0.clone().double()
    ref.moe_combine(eh, y.cpu(), cplan.row_of, gates)
    close(h, eh, 1e-5, 1e-5)
    # dense gated product (one "expert")
    d = torch.empty(T, I, dtype=dtype, device=DEV)
    ops.gated_gemm(x.to(DEV), w13[0].to(DEV), d, act)
    ed = torch.zeros(T, I, dtype=torch.float64)
    ref.gated_gemm(x, r13[0], ed, act)
    close(d, ed, *tol)
    # few rows: the split path (plain product over the paired rows, then the activation)
    for rows in (1, 9):
        ids_s = ids[:rows].contiguous()
        plan_s = ops.moe_plan(ids_s.to(DEV), E, ops.moe_tile_rows(rows, E, dtype))
        xs_s = torch.empty(2 * rows, H, dtype=dtype, device=DEV)
        ops.gather_rows(x.to(DEV), plan_s.token_of, xs_s)
        a_s = torch.empty(2 * rows, I, dtype=dtype, device=DEV)
        ops.gated_gemm(xs_s, w13.to(DEV), a_s, act, plan_s)
        cp = MoePlan(E, plan_s.tile_rows, plan_s.max_tiles, *(t.cpu() for t in (plan_s.counts, plan_s.offsets, plan_s.row_of,
                     plan_s.token_of, plan_s.tile_expert, plan_s.tile_row0, plan_s.n_tiles)))
        ea_s = torch.zeros(2 * rows, I, dtype=torch.float64)
        ref.gated_gemm(xs_s.cpu(), r13, ea_s, act, cp)
        close(a_s, ea_s, *tol)
        # the down product left as partial slices (the K blocks of all tiles cut into equal runs)
        yp = ops.gemm_partials(a_s, w2.to(DEV), plan=plan_s)
        assert yp.dim() == 3 and tuple(yp.shape[1:]) == (2 * rows, H)
        ey_s = torch.zeros(2 * rows, H, dtype=torch.float64)
        ref.grouped_gemm(a_s.cpu(), w2, ey_s, cp)
        close(yp.sum(0), ey_s, 1e-5, 1e-5)


@pytest.mark.parametrize("tile", [128, 256])
def test_gated_and_grouped_wide_tiles(ops, ref, tile):
    """Many rows per expert: full tiles, tiles cut short by the end of an expert's rows, an expert with few rows."""
    from flint_b200.csrc.ops import MoePlan
    T, H, I, E = 900, 192, 136, 3
    ids = torch.zeros(T, 2, dtype=torch.int32)
    ids[:, 0] = torch.randint(0, 2, (T,), dtype=torch.int32)       # experts 0 and 1 share most rows
    ids[:, 1] = torch.where(torch.arange(T) % 90 == 0, 2, 1 - ids[:, 0]).to(torch.int32)   # expert 2: ten rows
    plan = ops.moe_plan(ids.to(DEV), E, tile)
    x = rnd(T, H, dtype=torch.bfloat16)
    xs = torch.empty(2 * T, H, dtype=torch.bfloat16, device=DEV)
    ops.gather_rows(x.to(DEV), plan.token_of, xs)
    w1, w3, w2 = (rnd(E, I, H, dtype=torch.bfloat16, seed=1, scale=0.1), rnd(E, I, H, dtype=torch.bfloat16, seed=2, scale=0.1),
                  rnd(E, H, I, dtype=torch.bfloat16, seed=3, scale=0.1))
    a = torch.full((2 * T, I), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.gated_gemm(xs, ops.pair_gate_up(w1, w3).contiguous().to(DEV), a, "silu", plan)
    cplan = MoePlan(E, tile, plan.max_tiles, *(t.cpu() for t in (plan.counts, plan.offsets, plan.row_of, plan.token_of,
                                                               plan.tile_expert, plan.tile_row0, plan.n_tiles)))
    ea = torch.zeros(2 * T, I, dtype=torch.float64)
    ref.gated_gemm(xs.cpu(), ref.pair_gate_up(w1, w3), ea, "silu", cplan)
    close(a, ea, 2e-2, 2e-2)
    y = torch.empty(2 * T, H, device=DEV)
    ops.grouped_gemm(a, w2.to(DEV), y, plan)
    ey = torch.zeros(2 * T, H, dtype=torch.float64)
    ref.grouped_gemm(a.cpu(), w2, ey, cplan)
    close(y, ey, 1e-4, 1e-4)


@pytest.mark.parametrize("wd", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,E,eps", [(50, 96, 6, 0.05), (9, 1000, 16, 0.01), (33, 64, 4, 0.3), (4, 40, 3, 0.01)])
def test_router_sparsemixer(ops, ref, wd, T, H, E, eps):
    x, wr = rnd(T, H), rnd(E, H, dtype=wd, seed=1, scale=0.3)
    # hand-made rows: a tie for the maximum, a negative maximum, a runner-up inside the mask band
    tie = torch.zeros(H); x[0] = tie
    ids, gates = torch.empty(T, 2, dtype=torch.int32, device=DEV), torch.empty(T, 2, device=DEV)
    lg = torch.empty(T, E, device=DEV)
    ops.router_sparsemixer(x.to(DEV), wr.to(DEV), eps, ids, gates, lg)
    eids, egates, elg = torch.empty(T, 2, dtype=torch.int32), torch.empty(T, 2, dtype=torch.float64), torch.empty(T, E, dtype=torch.float64)
    RefOps(torch.float64).router_sparsemixer(x, wr, eps, eids, egates, elg)
    close(lg, elg, 1e-5, 1e-5)
    assert torch.equal(ids.cpu(), eids)
    close(gates, egates, 1e-4, 1e-5)
    assert ids.cpu()[0].tolist() == [0, 1]      # ties go to the lowest index


def test_sparsemixer_by_hand(ops):
    """Router logits chosen by an identity-like weight so that the selection can be checked by hand:
    s = [2, 1.9, -1, 0.5], eps 0.1 -> threshold 0.2.  First pick 0; (2-1.9)/2=0.05 keeps 1, others
    masked: g1 = 1/(1+e^-0.1).  Second pick 1 (m2=1.9): (1.9-0.5)/1.9 > 0.2 masked, (1.9+1)/1.9 masked:
    g2 = 1."""
    H, E = 8, 4
    wr = torch.zeros(E, H); wr[0, 0] = wr[1, 1] = wr[2, 2] = wr[3, 3] = 1.0
    x = torch.zeros(2, H); x[0, :4] = torch.tensor([2.0, 1.9, -1.0, 0.5])
    x[1, :4] = torch.tensor([-3.0, -1.0, -1.05, -2.0])   # negative maximum: factor = |s|
    ids, gates = torch.empty(2, 2, dtype=torch.int32, device=DEV), torch.empty(2, 2, device=DEV)
    ops.router_sparsemixer(x.to(DEV), wr.to(DEV), 0.1, ids, gates)
    assert ids.cpu().tolist() == [[0, 1], [1, 2]]
    g = gates.cpu()
    assert abs(g[0, 0].item() - 1 / (1 + math.exp(-0.1))) < 1e-6 and abs(g[0, 1].item() - 1.0) < 1e-6
    # row 1: m1=-1: (-1+1.05)/1.05=0.0476 keeps 2; (-1+2)/2=.5, (-1+3)/3=.67 masked -> g1=1/(1+e^-0.05)
    assert abs(g[1, 0].item() - 1 / (1 + math.exp(-0.05))) < 1e-6
    # second pick 2 (m2=-1.05): (-1.05+2)/2=.475 masked, (-1.05+3)/3=.65 masked -> g2 = 1
    assert abs(g[1, 1].item() - 1.0) < 1e-6


def make_cache(n_pages, nkv, P, hd, dtype, slots, max_pages, seed=0):
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(n_pages, nkv, P, hd, generator=g).to(dtype)
    v = torch.randn(n_pages, nkv, P, hd, generator=g).to(dtype)
    bt = torch.full((slots, max_pages), -1, dtype=torch.int32)
    return k, v, bt


def views(k, v, bt, P, nkv, hd, window):
    spec = KVSpec(nkv, hd, window)
    return (CacheView(k.to(DEV), v.to(DEV), bt.to(DEV), P, spec), CacheView(k.clone(), v.clone(), bt.clone(), P, spec))


@pytest.mark.parametrize("qd,cd", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("nq,nkv,hd,P,window", [(4, 2, 16, 16, 0), (3, 1, 32, 16, 48), (6, 1, 48, 32, 0),
                                                 (32, 8, 128, 64, 0), (5, 5, 80, 16, 20), (16, 2, 256, 16, 0)])
def test_rope_write_and_attention(ops, ref, qd, cd, nq, nkv, hd, P, window):
    slots, max_pages, n_pages = 3, 12, 30
    k, v, bt = make_cache(n_pages, nkv, P, hd, cd, slots, max_pages)
    # scattered pages: slot 0 holds 150 positions, slot 2 holds 37
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(5)).to(torch.int32)
    bt[0, :10] = perm[:10]; bt[2, :3] = perm[10:13]
    lens = {0: min(150, 10 * P), 2: min(37, 3 * P)}
    dv, cv = views(k, v, bt, P, nkv, hd, window)
    # rows: a portion of slot 0 ending at its last position, and one decoded token of slot 2
    n0 = 23
    pos = torch.tensor(list(range(lens[0] - n0, lens[0])) + [lens[2] - 1], dtype=torch.int32)
    slot = torch.tensor([0] * n0 + [2], dtype=torch.int32)
    T = pos.numel()
    rot = hd if hd != 80 else 48
    maxpos = 256
    ang = torch.arange(maxpos, dtype=torch.float64)[:, None] * (10000.0 ** (-torch.arange(rot // 2, dtype=torch.float64) * 2 / rot))
    cos, sin = (torch.cos(ang) * 1.2).float(), (torch.sin(ang) * 1.2).float()
    qkv = rnd(T, (nq + 2 * nkv) * hd)
    q_d = torch.empty(T, nq * hd, dtype=qd, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.rope_kv_write(qkv.to(DEV), pos.to(DEV), slot.to(DEV), cos.to(DEV), sin.to(DEV), rot, q_d, dv, nq, nkv, hd, True, status)
    q_r = torch.empty(T, nq * hd, dtype=torch.float64)
    ref.rope_kv_write(qkv, pos, slot, cos, sin, rot, q_r, cv, nq, nkv, hd, True, None)
    assert int(status.item()) == 0
    tol = (1e-6, 1e-6) if qd == torch.float32 else (1e-2, 1e-2)
    close(q_d, q_r, *tol)
    close(dv.k, cv.k, *((1e-6, 1e-6) if cd == torch.float32 else (1e-2, 1e-2)))
    close(dv.v, cv.v, 0, 0)
    # make one far key stand out for row 0 of slot 0, so that a kernel that skips it is caught
    out_d = torch.empty(T, nq * hd, dtype=qd, device=DEV)
    scale = 1 / math.sqrt(hd)
    span = min(lens[0], window or 10 ** 9)
    for kernel, splits in (("warp", None), ("warp", (32, -(-span // 32))), ("warp", (64, -(-span // 64))), ("block", None),
                           ("block", (128, -(-span // 128))), ("block", (span, 1)), ("block", (40, -(-span // 40))),
                           ("tma", None), ("tma", (span, 1)), ("tma", (48, -(-span // 48))), ("tma", (23, -(-span // 23)))):
        if kernel == "tma" and (hd > 128 or qd != torch.bfloat16):
            continue
        out_d.fill_(float("nan"))
        ops.paged_attention(q_d, dv, pos.to(DEV), slot.to(DEV), out_d, nq, nkv, hd, window, scale, max(lens.values()),
                            splits=splits, kernel=kernel)
        out_r = torch.empty(T, nq * hd, dtype=torch.float64)
        # the reference reads the device's cache content (bf16-rounded where it is) and the device's q
        cv2 = CacheView(dv.k.cpu(), dv.v.cpu(), bt, P, dv.spec)
        ref.paged_attention(q_d.cpu(), cv2, pos, slot, out_r, nq, nkv, hd, window, scale, max(lens.values()))
        close(out_d, out_r, *((2e-5, 2e-5) if qd == torch.float32 else (2e-2, 2e-2)))


@pytest.mark.parametrize("rot", [8, 32])
def test_rope_write_with_neighbouring_dims_rotating_together(ops, ref, rot):
    """The other rotation style (dims 2i and 2i + 1), with split partial sums, a bias and the cache write."""
    T, nq, nkv, hd, P = 7, 4, 2, 32, 16
    W = (nq + 2 * nkv) * hd
    parts = rnd(3, T, W)
    bias = rnd(W, seed=5)
    k, v, bt = make_cache(4, nkv, P, hd, torch.float32, 2, 4)
    bt[0, :2] = torch.tensor([3, 1], dtype=torch.int32)
    bt[1, :1] = torch.tensor([0], dtype=torch.int32)
    dv, cv = views(k, v, bt, P, nkv, hd, 0)
    pos = torch.tensor([10, 11, 12, 13, 14, 0, 1], dtype=torch.int32)
    slot = torch.tensor([0, 0, 0, 0, 0, 1, 1], dtype=torch.int32)
    ang = torch.arange(32, dtype=torch.float64)[:, None] * (100.0 ** (-torch.arange(rot // 2, dtype=torch.float64) * 2 / rot))
    cos, sin = torch.cos(ang).float(), torch.sin(ang).float()
    q_d = torch.empty(T, nq * hd, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.rope_kv_write(parts.to(DEV), pos.to(DEV), slot.to(DEV), cos.to(DEV), sin.to(DEV), rot, q_d, dv, nq, nkv, hd, True,
                      status, bias=bias.to(DEV), style="interleaved")
    q_r = torch.empty(T, nq * hd, dtype=torch.float64)
    ref.rope_kv_write(parts, pos, slot, cos, sin, rot, q_r, cv, nq, nkv, hd, True, None, bias=bias, style="interleaved")
    close(q_d, q_r, 1e-5, 1e-5)
    close(dv.k, cv.k, 1e-5, 1e-5)
    close(dv.v, cv.v, 1e-5, 1e-5)
    # by hand for one element pair: (x0, x1) of head 0 of token 0 rotate by the angle of position 10, pair 0
    x = parts.double().sum(0)[0] + bias.double()
    c, s_ = math.cos(10.0), math.sin(10.0)
    assert abs(q_d[0, 0].item() - (x[0] * c - x[1] * s_).item()) < 1e-4
    assert abs(q_d[0, 1].item() - (x[1] * c + x[0] * s_).item()) < 1e-4
    assert int(status.item()) == 0


def test_attention_far_key_stands_out(ops, ref):
    """One key far back among hundreds gets a large score: the output must be (almost) its value."""
    nq, nkv, hd, P = 2, 1, 32, 16
    n_pages, L = 40, 600
    k, v, bt = make_cache(n_pages, nkv, P, hd, torch.float32, 1, 40, seed=3)
    k *= 0.05
    bt[0, :38] = torch.arange(38, dtype=torch.int32).flip(0)
    far = 3
    q = rnd(1, nq * hd) * 0.05
    k[bt[0, far // P].long(), 0, far % P] = q[0, :hd] * 4000.0      # head 0's query matches this key
    dv, cv = views(k, v, bt, P, nkv, hd, 0)
    pos, slot = torch.tensor([L - 1], dtype=torch.int32), torch.tensor([0], dtype=torch.int32)
    out = torch.empty(1, nq * hd, device=DEV)
    for kernel, splits in (("warp", None), ("warp", (32, 19)), ("warp", (600, 1)), ("block", None), ("block", (256, 3))):
        ops.paged_attention(q.to(DEV), dv, pos.to(DEV), slot.to(DEV), out, nq, nkv, hd, 0, 1 / math.sqrt(hd), L,
                            splits=splits, kernel=kernel)
        exp = torch.empty(1, nq * hd, dtype=torch.float64)
        ref.paged_attention(q, cv, pos, slot, exp, nq, nkv, hd, 0, 1 / math.sqrt(hd), L)
        close(out, exp, 1e-4, 1e-5)
        close(out[0, :hd], v[bt[0, far // P].long(), 0, far % P], 1e-3, 1e-3)
    # with a window that ends just after the far key it must vanish; one position wider and it is back
    for kernel in ("warp", "block"):
        for window, present in ((L - 1 - far, False), (L - far, True)):
            ops.paged_attention(q.to(DEV), dv, pos.to(DEV), slot.to(DEV), out, nq, nkv, hd, window, 1 / math.sqrt(hd), L,
                                kernel=kernel)
            is_far = torch.allclose(out[0, :hd].cpu(), v[bt[0, far // P].long(), 0, far % P], atol=1e-3)
            assert is_far == present


@pytest.mark.parametrize("nq,nkv,hd,P,window,lens,portions", [
    (4, 2, 16, 16, 0, (100, 37), (100, 20)), (3, 1, 32, 16, 48, (300, 90), (200, 50)),
    (32, 8, 128, 64, 0, (700, 128), (300, 128)), (6, 2, 64, 32, 0, (257, 65), (129, 65)),
    (5, 5, 80, 64, 20, (150, 40), (100, 40)), (8, 2, 96, 128, 0, (300, 20), (260, 16)),
    (2, 2, 128, 16, 100, (500, 17), (130, 17))])
def test_attention_prefill_on_tensor_cores(ops, ref, nq, nkv, hd, P, window, lens, portions):
    """Tiles of long portions on the tcgen05 kernel, one decoded row of a third request beside them
    through the row list, all in one output buffer; scattered pages; portions that start deep in a
    request (keys of earlier portions come from the cache)."""
    g = torch.Generator().manual_seed(nq * 131 + hd)
    lens = (*lens, 77)
    need = [-(-n // P) for n in lens]
    n_pages = sum(need) + 3
    k = torch.randn(n_pages, nkv, P, hd, generator=g).to(torch.bfloat16)
    v = torch.randn(n_pages, nkv, P, hd, generator=g).to(torch.bfloat16)
    bt = torch.full((3, max(need) + 1), -1, dtype=torch.int32)
    perm = torch.randperm(n_pages, generator=g).to(torch.int32)
    o = 0
    for s_, n in enumerate(need):
        bt[s_, :n] = perm[o:o + n]
        o += n
    pos, slot, tiles = [], [], []
    for s_, (n_total, n_rows) in enumerate(zip(lens[:2], portions)):
        base = len(pos)
        pos += list(range(n_total - n_rows, n_total))
        slot += [s_] * n_rows
        for r in range(0, n_rows, 128):
            tiles += [base + r, min(128, n_rows - r), s_, n_total - n_rows + r]
    other = [len(pos)]
    pos.append(lens[2] - 1)
    slot.append(2)
    T = len(pos)
    pos, slot = torch.tensor(pos, dtype=torch.int32), torch.tensor(slot, dtype=torch.int32)
    q = torch.randn(T, nq * hd, generator=g).to(torch.bfloat16)
    spec = KVSpec(nkv, hd, window)
    dv = CacheView(k.to(DEV), v.to(DEV), bt.to(DEV), P, spec)
    out = torch.full((T, nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    scale = 1 / math.sqrt(hd)
    ops.attention_prefill_tc(q.to(DEV), dv, torch.tensor(tiles, dtype=torch.int32, device=DEV), len(tiles) // 4, out, nq,
                             nkv, hd, window, scale)
    assert torch.isnan(out[other[0]]).all() and not torch.isnan(out[:other[0]]).any()    # only its own rows
    ops.paged_attention(q.to(DEV), dv, pos.to(DEV), slot.to(DEV), out, nq, nkv, hd, window, scale, max(lens),
                        rows=torch.tensor(other, dtype=torch.int32, device=DEV))
    assert int(ops.tc_error.item()) == 0
    exp = torch.zeros(T, nq * hd, dtype=torch.float64)
    ref.paged_attention(q, CacheView(k, v, bt, P, spec), pos, slot, exp, nq, nkv, hd, window, scale, max(lens))
    close(out, exp, 2e-2, 2e-2)


@pytest.mark.parametrize("nq,nkv,hd,P,window,lens", [
    (8, 8, 128, 64, 0, (77,)),                                # one short row: items of 5 steps cut into runs of 3
    (32, 8, 128, 64, 0, (700, 128, 77, 1, 16, 17)),           # ragged: a run ends one item and begins the next
    (4, 2, 64, 16, 0, (300,)),
    (6, 2, 48, 32, 40, (500, 90, 41, 300)),                   # a window: the first step starts below the first visible key
    (16, 4, 128, 64, 0, tuple(300 + 7 * i for i in range(64))),   # many rows
])
def test_attention_decode_stream_cuts_keys_into_equal_runs(ops, ref, nq, nkv, hd, P, window, lens):
    """The decode kernel that divides the 16-key steps of all rows among its warps by itself, on rows of
    very different lengths, through a row list, with scattered pages."""
    g = torch.Generator().manual_seed(len(lens) * 31 + hd)
    need = [-(-n // P) for n in lens]
    n_pages = sum(need) + 2
    k = torch.randn(n_pages, nkv, P, hd, generator=g).to(torch.bfloat16)
    v = torch.randn(n_pages, nkv, P, hd, generator=g).to(torch.bfloat16)
    bt = torch.full((len(lens), max(need) + 1), -1, dtype=torch.int32)
    perm = torch.randperm(n_pages, generator=g).to(torch.int32)
    o = 0
    for s_, n in enumerate(need):
        bt[s_, :n] = perm[o:o + n]
        o += n
    T = len(lens)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    slot = torch.arange(T, dtype=torch.int32)
    q = torch.randn(T, nq * hd, generator=g).to(torch.bfloat16)
    spec = KVSpec(nkv, hd, window)
    dv = CacheView(k.to(DEV), v.to(DEV), bt.to(DEV), P, spec)
    scale = 1 / math.sqrt(hd)
    exp = torch.zeros(T, nq * hd, dtype=torch.float64)
    ref.paged_attention(q, CacheView(k, v, bt, P, spec), pos, slot, exp, nq, nkv, hd, window, scale, max(lens))
    out = torch.full((T, nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    for fresh_keys in (1 << 30, 1):      # 1: a decode step, the first tiles are fetched before the wait for the kernel before
        out.fill_(float("nan"))
        ops.paged_attention(q.to(DEV), dv, pos.to(DEV), slot.to(DEV), out, nq, nkv, hd, window, scale, max(lens),
                            kernel="stream", fresh_keys=fresh_keys)
        assert int(ops.tc_error.item()) == 0
        close(out, exp, 2e-2, 2e-2)
    if T > 2:       # every other row through a row list: the rest stays untouched
        rows = torch.arange(0, T, 2, dtype=torch.int32)
        out2 = torch.full((T, nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.paged_attention(q.to(DEV), dv, pos.to(DEV), slot.to(DEV), out2, nq, nkv, hd, window, scale, max(lens),
                            kernel="stream", rows=rows.to(DEV))
        assert torch.isnan(out2[1::2]).all()
        close(out2[0::2], exp[0::2], 2e-2, 2e-2)


@pytest.mark.parametrize("rows,n_keys,expect", [
    (8, 2049, "tma"), (18, 2049, "tma"), (20, 2049, "stream"), (24, 1600, "stream"), (31, 2049, "stream"),
    (24, 513, "tma"), (3, 16400, "stream"), (2, 16400, "tma"), (16, 3100, "stream"), (12, 3072, "tma"),
])
def test_attention_decode_of_even_batches_by_the_planned_kernel(ops, ref, rows, n_keys, expect):
    """Batches of decoded tokens of about equal length, the kernel and the cut chosen by the plan (not given):
    on either side of the lines where the plan changes kernels, the result is the reference's."""
    nq, nkv, hd, P = 32, 8, 128, 64
    if ops.sm_count == 148:          # the lines are where they were measured, on a device of 148 SMs
        assert ops.attention_plan(rows, nq, nkv, n_keys, hd, True, False)[0] == expect
    g = torch.Generator().manual_seed(rows * 7 + n_keys)
    lens = [n_keys - (i * 5) % 23 for i in range(rows)]            # about equal: within a few keys of each other
    need = [-(-n // P) for n in lens]
    n_pages = sum(need) + 2
    k = (torch.randn(n_pages, nkv, P, hd, generator=g) * 0.5).to(torch.bfloat16)
    v = torch.randn(n_pages, nkv, P, hd, generator=g).to(torch.bfloat16)
    bt = torch.full((rows, max(need) + 1), -1, dtype=torch.int32)
    perm = torch.randperm(n_pages, generator=g).to(torch.int32)
    o = 0
    for s_, n in enumerate(need):
        bt[s_, :n] = perm[o:o + n]
        o += n
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    slot = torch.arange(rows, dtype=torch.int32)
    q = (torch.randn(rows, nq * hd, generator=g) * 0.5).to(torch.bfloat16)
    spec = KVSpec(nkv, hd, 0)
    scale = 1 / math.sqrt(hd)
    exp = torch.zeros(rows, nq * hd, dtype=torch.float64)
    ref.paged_attention(q, CacheView(k, v, bt, P, spec), pos, slot, exp, nq, nkv, hd, 0, scale, max(lens))
    out = torch.full((rows, nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.paged_attention(q.to(DEV), CacheView(k.to(DEV), v.to(DEV), bt.to(DEV), P, spec), pos.to(DEV), slot.to(DEV), out,
                        nq, nkv, hd, 0, scale, max(lens), ragged=False, fresh_keys=1)
    assert int(ops.tc_error.item()) == 0
    close(out, exp, 2e-2, 2e-2)


@pytest.mark.parametrize("nq,nkv,hd,P,window,lens,splits", [
    (32, 8, 128, 64, 0, (2048, 2040, 1990, 2047), (128, 16)),     # four warps of a block merge, then the blocks of an item
    (32, 8, 128, 64, 0, (500, 512), (128, 4)),                    # four splits: the block writes the result itself
    (8, 1, 64, 16, 0, (300, 20), (64, 5)),                        # splits not in fours: merged by a kernel of its own
    (32, 8, 128, 64, 0, (4000,), (64, 64)),                       # sixteen records an item: merged eight at a time
    (6, 2, 80, 16, 0, (333,), (48, 8)),                           # three query heads per kv head, a head size between
    (5, 5, 128, 32, 100, (400, 90), (32, 4)),                     # one query head per kv head, a window
    (48, 2, 96, 64, 0, (700, 640, 1), (64, 12)),                  # 24 query heads per kv head: three chunks of eight
])
def test_attention_decode_splits_are_merged_by_the_last_to_arrive(ops, ref, nq, nkv, hd, P, window, lens, splits):
    """The decode kernel with a fixed cut of every row's key range: the pieces of a (row, kv head) are merged
    inside the kernel when they come in fours (the four warps of a block through shared memory, then the
    blocks of the item by the one that finishes last), or by a kernel of its own; both give the reference's
    result, and the arrival counters are zero again after every launch."""
    g = torch.Generator().manual_seed(len(lens) * 17 + hd + nq)
    need = [-(-n // P) for n in lens]
    n_pages = sum(need) + 2
    k = torch.randn(n_pages, nkv, P, hd, generator=g).to(torch.bfloat16)
    v = torch.randn(n_pages, nkv, P, hd, generator=g).to(torch.bfloat16)
    bt = torch.full((len(lens), max(need) + 1), -1, dtype=torch.int32)
    perm = torch.randperm(n_pages, generator=g).to(torch.int32)
    o = 0
    for s_, n in enumerate(need):
        bt[s_, :n] = perm[o:o + n]
        o += n
    T = len(lens)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    slot = torch.arange(T, dtype=torch.int32)
    q = torch.randn(T, nq * hd, generator=g).to(torch.bfloat16)
    spec = KVSpec(nkv, hd, window)
    dv = CacheView(k.to(DEV), v.to(DEV), bt.to(DEV), P, spec)
    scale = 1 / math.sqrt(hd)
    exp = torch.zeros(T, nq * hd, dtype=torch.float64)
    ref.paged_attention(q, CacheView(k, v, bt, P, spec), pos, slot, exp, nq, nkv, hd, window, scale, max(lens))
    outs = []
    for merge_in_kernel in (True, True, False):
        out = torch.full((T, nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        # fresh_keys=1: only a row's own key may be written by the kernel before (a decode step), so the first
        # tiles are fetched before the wait for that kernel
        ops.paged_attention(q.to(DEV), dv, pos.to(DEV), slot.to(DEV), out, nq, nkv, hd, window, scale, max(lens),
                            kernel="tma", splits=splits, merge_in_kernel=merge_in_kernel,
                            fresh_keys=1 if merge_in_kernel else 1 << 30)
        assert int(ops.tc_error.item()) == 0 and int(ops.attention_arrivals.abs().sum().item()) == 0
        close(out, exp, 2e-2, 2e-2)
        outs.append(out.float().cpu())
    assert torch.equal(outs[0], outs[1])
    close(outs[0], outs[2].double(), 1e-2, 1e-2)


@pytest.mark.parametrize("ramp", [0.02, 0.3])
def test_attention_prefill_growing_scores(ops, ref, ramp):
    """Keys aligned with the queries and growing with their position: a row's maximum keeps rising, slowly
    (the softmax reference stays behind it for many tiles) or fast (it moves at every tile, and the output
    kept on the chip is rescaled); and one late key that stands out for the rows after it."""
    nq, nkv, hd, P, L = 2, 1, 64, 64, 640
    g = torch.Generator().manual_seed(5)
    n_pages = L // P
    direction = torch.randn(hd, generator=g)
    direction /= direction.norm()
    k = (torch.randn(n_pages, nkv, P, hd, generator=g) * 0.3)
    key_pos = torch.arange(L).view(n_pages, 1, P, 1)
    k += direction * ramp * key_pos                      # score of key j grows like ramp * j * |q . direction|
    v = torch.randn(n_pages, nkv, P, hd, generator=g)
    q = torch.randn(L, nq * hd, generator=g) * 0.3
    q[:, :hd] += direction * 4.0
    q[:, hd:] += direction * 4.0
    late = 500
    k.view(-1, hd)[late] = direction * 400.0 * (1 if ramp < 0.1 else 3)
    k, v, q = k.to(torch.bfloat16), v.to(torch.bfloat16), q.to(torch.bfloat16)
    bt = torch.arange(n_pages, dtype=torch.int32).flip(0).view(1, -1).contiguous()
    k_paged, v_paged = k.flip(0).contiguous(), v.flip(0).contiguous()      # logical page i sits in page n-1-i
    pos, slot = torch.arange(L, dtype=torch.int32), torch.zeros(L, dtype=torch.int32)
    tiles = []
    for r in range(0, L, 128):
        tiles += [r, min(128, L - r), 0, r]
    spec = KVSpec(nkv, hd, 0)
    out = torch.empty(L, nq * hd, dtype=torch.bfloat16, device=DEV)
    scale = 1 / math.sqrt(hd)
    ops.attention_prefill_tc(q.to(DEV), CacheView(k_paged.to(DEV), v_paged.to(DEV), bt.to(DEV), P, spec),
                             torch.tensor(tiles, dtype=torch.int32, device=DEV), len(tiles) // 4, out, nq, nkv, hd, 0, scale)
    assert int(ops.tc_error.item()) == 0
    exp = torch.zeros(L, nq * hd, dtype=torch.float64)
    ref.paged_attention(q, CacheView(k_paged, v_paged, bt, P, spec), pos, slot, exp, nq, nkv, hd, 0, scale, L)
    close(out, exp, 2e-2, 2e-2)
    # rows after the late key see (almost) only its value
    close(out[late + 1, :hd], v.view(-1, hd)[late].double(), 2e-2, 2e-2)


@pytest.mark.parametrize("R,V", [(1, 17), (5, 1000), (3, 32064)])
def test_argmax(ops, R, V):
    lg = rnd(R, V)
    lg[0, 3] = lg[0, min(7, V - 1)] = 100.0        # first maximum wins
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    ops.argmax(lg.to(DEV), out)
    assert out.cpu().tolist() == torch.argmax(lg, -1).tolist()
    assert out.cpu()[0].item() == 3


@pytest.mark.parametrize("nq,nkv,hd,P,window,lens,rot,slices", [
    (32, 8, 128, 64, 0, (2049, 2040, 2030, 2048, 2047, 2046, 2001, 2049), 128, 9),   # a batch of eight at the measured sizes
    (32, 8, 128, 64, 0, (2049,), 128, 9),                                         # one row: stages of 32 keys
    (8, 2, 64, 16, 0, (300, 290, 310), 32, 3),                                    # part of the head rotates
    (6, 2, 48, 16, 40, (100, 90, 95), 16, 1),                                     # a window, three query heads per kv head
    (48, 2, 96, 64, 0, (700, 690), 96, 2),                                        # 24 query heads per kv head: three chunks
    (4, 4, 16, 16, 0, (5, 6, 7, 6), 16, 2),                                       # rows shorter than one split
    (32, 8, 128, 64, 0, (1, 1), 128, 4),                                          # first tokens: nothing cached yet
    (8, 2, 128, 32, 0, (65, 64, 63), 0, 2),                                       # no rotation at all, a page's edge
])
def test_rotary_write_and_decode_attention_in_one_kernel(ops, ref, nq, nkv, hd, P, window, lens, rot, slices):
    """The decode kernel that also sums the projection's partial slices, adds the bias, rotates q and k, writes the
    rows' new keys and values into their pages and uses them itself: the same output and the same cache content
    as the rotary kernel followed by attention, computed in float64."""
    g = torch.Generator().manual_seed(nq * 7 + hd + len(lens))
    T = len(lens)
    need = [-(-n // P) for n in lens]
    n_pages = sum(need) + 2
    k = torch.randn(n_pages, nkv, P, hd, generator=g).to(torch.bfloat16)
    v = torch.randn(n_pages, nkv, P, hd, generator=g).to(torch.bfloat16)
    bt = torch.full((T, max(need) + 1), -1, dtype=torch.int32)
    perm = torch.randperm(n_pages, generator=g).to(torch.int32)
    o = 0
    for s_, n in enumerate(need):
        bt[s_, :n] = perm[o:o + n]
        o += n
    W = (nq + 2 * nkv) * hd
    parts = torch.randn(slices, T, W, generator=g) * 0.6
    bias = torch.randn(W, generator=g) * 0.3
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    slot = torch.arange(T, dtype=torch.int32)
    half = max(rot // 2, 1)
    ang = torch.arange(max(lens) + 1, dtype=torch.float64)[:, None] * (10000.0 ** (-torch.arange(half, dtype=torch.float64) / half))
    cos, sin = (torch.cos(ang) * 1.1).float(), (torch.sin(ang) * 1.1).float()
    spec = KVSpec(nkv, hd, window)
    dv = CacheView(k.to(DEV), v.to(DEV), bt.to(DEV), P, spec)
    cv = CacheView(k.clone(), v.clone(), bt.clone(), P, spec)
    scale = 1 / math.sqrt(hd)
    # the reference: rotary write, then attention over the cache as the write left it
    q_r = torch.empty(T, nq * hd, dtype=torch.float64)
    ref.rope_kv_write(parts, pos, slot, cos, sin, rot, q_r, cv, nq, nkv, hd, True, None, bias=bias)
    exp = torch.zeros(T, nq * hd, dtype=torch.float64)
    ref.paged_attention(q_r.to(torch.bfloat16), cv, pos, slot, exp, nq, nkv, hd, window, scale, max(lens))

    class Step:
        pass
    step = Step()
    step.pos, step.slot, step.n_tokens, step.entries = pos.to(DEV), slot.to(DEV), T, [None] * T
    step.max_kv_len, step.even_lengths, step.attention_splits = max(lens), True, None
    step.status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full((T, nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    for _ in range(2):                   # twice: the second launch finds the first one's keys in the pages already
        done = ops.rope_attention_decode(parts.to(DEV), bias.to(DEV), cos.to(DEV), sin.to(DEV), rot, "half", dv, step, out,
                                         nq, nkv, hd, window, scale)
        assert done
        assert int(ops.tc_error.item()) == 0 and int(step.status.item()) == 0
        assert int(ops.attention_arrivals.abs().sum().item()) == 0
        close(out, exp, 2e-2, 2e-2)
        close(dv.k, cv.k, 1e-2, 1e-2)
        close(dv.v, cv.v, 1e-2, 1e-2)
    # a row whose page is missing raises the flag and writes nothing outside its pages
    bt2 = bt.clone()
    bt2[0, (lens[0] - 1) // P] = -1
    dv2 = CacheView(dv.k, dv.v, bt2.to(DEV), P, spec)
    ops.rope_attention_decode(parts.to(DEV), bias.to(DEV), cos.to(DEV), sin.to(DEV), rot, "half", dv2, step, out, nq, nkv,
                              hd, window, scale)
    assert int(step.status.item()) == 1
