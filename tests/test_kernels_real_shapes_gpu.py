"""The tensor-core products at exactly the shapes the engine is measured at (Phi-mini-MoE and Phi-3.5-MoE layer
sizes), against float64: the K loop of 64 blocks through the ring over several persistent items, the K splits the
launch planner picks, the vocabulary's ragged last tile, and the expert products both as stream-K partial slices
(few rows) and as 256-row tiles (many rows) with expert widths of 960 and 6,400."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from flint_b200.csrc.ops import get_ops
    return get_ops(DEV)


def device_randn(*shape, seed, scale):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(*shape, generator=g, device=DEV) * scale).to(torch.bfloat16)


def close(got, want, rtol, atol, what):
    err = (got.double().cpu() - want).abs()
    bound = atol + rtol * want.abs()
    assert torch.isfinite(got).all(), what
    assert (err <= bound).all(), f"{what}: max error {err.max().item():.3e}, worst excess {(err - bound).max().item():.3e}"


@pytest.mark.parametrize("rows", [1, 8, 64, 2048])
@pytest.mark.parametrize("N,K", [(6144, 4096), (4096, 4096), (32064, 4096)])
def test_dense_products_at_the_measured_shapes(ops, rows, N, K):
    x = device_randn(rows, K, seed=rows + N, scale=1.0)
    w = device_randn(N, K, seed=N + 1, scale=0.02)
    bias = torch.randn(N, device=DEV) * 0.1
    want = x.double().cpu() @ w.double().cpu().T
    # left as partial sums over the pieces of K that the planner picks (q/k/v and output projections)
    parts = ops.gemm_partials(x, w)
    assert tuple(parts.shape[1:]) == (rows, N)
    close(parts.sum(0), want, 1e-4, 2e-4, f"{parts.shape[0]} partial sums")
    # finished, with the bias (the output head)
    out = torch.empty(rows, N, device=DEV)
    ops.gemm(x, w, out, bias=bias)
    close(out, want + bias.double().cpu(), 1e-4, 2e-4, "finished product")
    out16 = torch.empty(rows, N, device=DEV, dtype=torch.bfloat16)
    ops.gemm(x, w, out16)
    close(out16, want, 1e-2, 1e-2, "bfloat16 output")
    assert int(ops.tc_error.item()) == 0


@pytest.mark.parametrize("T", [1, 8, 64, 2048])
@pytest.mark.parametrize("I", [960, 6400])
def test_expert_products_at_the_measured_shapes(ops, T, I):
    H, E = 4096, 16
    g = torch.Generator().manual_seed(T + I)
    first = torch.randint(0, E, (T,), generator=g)
    second = (first + 1 + torch.randint(0, E - 1, (T,), generator=g)) % E
    ids = torch.stack([first, second], 1).to(torch.int32).to(DEV)
    x = device_randn(T, H, seed=T, scale=1.0)
    w1 = device_randn(E, I, H, seed=1, scale=0.02)
    w3 = device_randn(E, I, H, seed=2, scale=0.02)
    w2 = device_randn(E, H, I, seed=3, scale=0.02)
    w13 = ops.pair_gate_up(w1, w3).contiguous()
    plan, xs = ops.moe_dispatch(ids, E, ops.moe_tile_rows(T, E, torch.bfloat16), x)
    a = torch.empty(2 * T, I, dtype=torch.bfloat16, device=DEV)
    ops.gated_gemm(xs, w13, a, "silu", plan)
    y = torch.empty(2 * T, H, device=DEV)
    ops.grouped_gemm(a, w2, y, plan)
    assert int(ops.tc_error.item()) == 0
    off = plan.offsets.cpu().tolist()
    token_of = plan.token_of.cpu().long()
    assert torch.equal(xs.cpu(), x.cpu()[token_of])
    want_a = torch.zeros(2 * T, I, dtype=torch.float64)
    want_y = torch.zeros(2 * T, H, dtype=torch.float64)
    a_host = a.double().cpu()
    for e in range(E):
        r0, r1 = off[e], off[e + 1]
        if r1 == r0:
            continue
        xe = xs[r0:r1].double().cpu()
        gate = xe @ w1[e].double().cpu().T
        want_a[r0:r1] = gate / (1 + torch.exp(-gate)) * (xe @ w3[e].double().cpu().T)
        want_y[r0:r1] = a_host[r0:r1] @ w2[e].double().cpu().T       # from the engine's own rounded activations
    close(a, want_a, 1e-2, 2e-3, "gate/up product")
    close(y, want_y, 1e-4, 2e-4, "down product")
