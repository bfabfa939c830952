"""Feed-forward parts: a dense gated MLP and a top-2 sparsemixer mixture of experts.

Dense: h += (act(x Wg^T) * (x Wu^T)) Wd^T, as the reference's feed-forward
(crates/thuban_model/src/ops/mlp.rs:24-79).  Mixture of experts (no counterpart in
the reference): float32 router logits, sparsemixer top-2 selection, rows sorted by
expert, two grouped products, and the gated sum of the two experts' outputs added to
the residual stream in a fixed order.
"""
from __future__ import annotations

import torch

from ..errors import ConfigError
from ..registry import FEED_FORWARDS
from .base import FeedForward, Pending, RouterRequest, mat, matmul_dtype


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(FeedForward):
    """params: hidden_size, intermediate_size, act; tensors gate_proj/up_proj [I,H], down_proj [H,I]."""

    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])
        self.act = params.get("act", "silu")

    def weights(self):
        return {"gate_proj.weight": mat(self.inter, self.hidden), "up_proj.weight": mat(self.inter, self.hidden),
                "down_proj.weight": mat(self.hidden, self.inter)}

    def fused(self):
        return {"gate_up_proj.weight": ["gate_proj.weight", "up_proj.weight"]}

    def load(self, t):
        dt = matmul_dtype(*t.values())
        # gate and up rows in the layout the kernels want: one product gives both
        self.w_gate_up = self.ops.pair_gate_up(t["gate_proj.weight"].to(dt), t["up_proj.weight"].to(dt)).contiguous()
        self.w_down = t["down_proj.weight"].to(dt)

    def input_dtypes(self):
        return (self.w_gate_up.dtype,)

    def forward(self, x, residual, step):
        xin = x[self.w_gate_up.dtype]
        a = torch.empty((xin.shape[0], self.inter), dtype=self.w_gate_up.dtype, device=xin.device)
        self.ops.gated_gemm(xin, self.w_gate_up, a, self.act)
        self.ops.gemm(a, self.w_down, residual, accumulate=True)


@FEED_FORWARDS.register("sparsemixer_moe")
class SparseMixerMoE(FeedForward):
    """params: hidden_size, intermediate_size, num_experts, jitter_eps, act.
    tensors: gate.weight [E,H]; experts.{e}.w1 / w3 [I,H] (gate / up), w2 [H,I] (down)."""

    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])
        self.E = int(params["num_experts"])
        if not 2 <= self.E <= 256:
            raise ConfigError(f"num_experts {self.E} is not supported (2..256)")
        self.eps = float(params["jitter_eps"])
        self.act = params.get("act", "silu")

    def weights(self):
        w = {"gate.weight": mat(self.E, self.hidden)}
        for e in range(self.E):
            w[f"experts.{e}.w1.weight"] = mat(self.inter, self.hidden)
            w[f"experts.{e}.w2.weight"] = mat(self.hidden, self.inter)
            w[f"experts.{e}.w3.weight"] = mat(self.inter, self.hidden)
        return w

    def load(self, t):
        self.w_router = t["gate.weight"]
        dt = matmul_dtype(*(t[k] for k in t if k.startswith("experts.")))
        # per expert the gate rows (w1) and the up rows (w3) in the layout the kernels want: [E, rows, H]
        self.w13 = torch.stack([self.ops.pair_gate_up(t[f"experts.{e}.w1.weight"].to(dt), t[f"experts.{e}.w3.weight"].to(dt))
                                for e in range(self.E)], 0).contiguous()
        self.w2 = torch.stack([t[f"experts.{e}.w2.weight"].to(dt) for e in range(self.E)], 0).contiguous()

    def input_dtypes(self):
        return (torch.float32, self.w13.dtype)

    def router_request(self, n_rows):
        """Routing can ride on the norm before this part (the normalised row is in registers there)."""
        dev = self.w_router.device
        return RouterRequest(self.w_router, self.eps, torch.empty((n_rows, 2), dtype=torch.int32, device=dev),
                             torch.empty((n_rows, 2), dtype=torch.float32, device=dev))

    def input_dtypes_when_routed(self):
        return (self.w13.dtype,)

    def forward(self, x, residual, step, routed=None):
        ops = self.ops
        xa = x[self.w13.dtype]
        T = xa.shape[0]
        dev = xa.device
        if routed is not None:
            ids, gates, logits = routed.expert_ids, routed.gates, routed.logits
        else:
            ids = torch.empty((T, 2), dtype=torch.int32, device=dev)
            gates = torch.empty((T, 2), dtype=torch.float32, device=dev)
            logits = torch.empty((T, self.E), dtype=torch.float32, device=dev) if step.record is not None else None
            ops.router_sparsemixer(x[torch.float32], self.w_router, self.eps, ids, gates, logits)
        plan, xs = ops.moe_dispatch(ids, self.E, ops.moe_tile_rows(T, self.E, self.w13.dtype), xa)
        a = torch.empty((2 * T, self.inter), dtype=self.w13.dtype, device=dev)
        ops.gated_gemm(xs, self.w13, a, self.act, plan)
        y = torch.empty((2 * T, self.hidden), dtype=torch.float32, device=dev)
        ops.grouped_gemm(a, self.w2, y, plan, plan_ready=True)     # the gate/up product ran over the same plan
        if step.record is not None:
            step.record.setdefault("experts", []).append(ids)
            step.record.setdefault("gates", []).append(gates)
            if logits is not None:
                step.record.setdefault("router_logits", []).append(logits)
        # the gated sum of the two experts' rows is added by the next norm's kernel
        return Pending(y=y, row_of=plan.row_of, gates=gates)
