"""Norm parts: LayerNorm (with or without bias) and RMSNorm.

LayerNorm: y = (x - mean) * rsqrt(var + eps) * gamma + beta with var = mean((x-mean)^2);
RMSNorm: y = x * rsqrt(mean(x^2) + eps) * gamma.  Statistics are float32.  The
reference's norm shader has both as modes (crates/thuban_kernel/wgsl/norm.wgsl:66-83,
112-121) and picks by config key (crates/thuban_architectures/src/phi.rs:55-63).
"""
from __future__ import annotations

import torch

from ..registry import NORMS
from .base import Norm, vec


class _RowNorm(Norm):
    mode = "layer"
    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.width = int(params["width"])
        self.eps = float(params["eps"])
        self.has_bias = bool(params.get("bias", False))
        self.gamma = self.beta = None

    def weights(self):
        w = {"weight": vec(self.width, init="gamma")}
        if self.has_bias:
            w["bias"] = vec(self.width)
        return w

    def load(self, tensors):
        self.gamma = tensors["weight"]
        self.beta = tensors.get("bias")

    supports_pending = True
    supports_router = True

    def forward(self, x, want, row_index=None, pending=None, router=None):
        rows = row_index.numel() if row_index is not None else x.shape[0]
        out = {}
        for dt in set(want):
            out[dt] = torch.empty((rows, self.width), dtype=dt, device=x.device)
        self.ops.row_norm(x, self.gamma, self.beta, self.eps, self.mode, out_f32=out.get(torch.float32),
                          out_bf16=out.get(torch.bfloat16), row_index=row_index, pending=pending, router=router)
        return out


@NORMS.register("layernorm")
class LayerNorm(_RowNorm):
    mode = "layer"


@NORMS.register("rmsnorm")
class RMSNorm(_RowNorm):
    mode = "rms"

    def __init__(self, params, ctx):
        super().__init__({**params, "bias": False}, ctx)
