"""The attention mixer: grouped-query attention over the paged cache.

q/k/v projection (one product over the concatenated weights, bias in its epilogue),
rotary encoding of q and k fused with the write of k and v into the cache pages,
attention of every row over its request's cached keys (causal, optionally windowed,
scale 1/sqrt(head_dim) unless given), and the output projection accumulated into the
residual stream.  Order of operations as the reference's dense decoder
(crates/thuban_architectures/src/transformer/forward.rs:114-365).
"""
from __future__ import annotations

import math

import torch

from ..cache.manager import KVSpec
from ..engine.step import StepNeeds
from ..errors import ConfigError, ModelError
from ..registry import MIXERS, POSITION_ENCODINGS
from .base import Mixer, Pending, mat, matmul_dtype, vec


def shared_position_encoding(spec, ctx):
    """One position-encoding object per distinct spec in a model."""
    key = ("position", spec.kind, repr(sorted(spec.params.items(), key=lambda kv: kv[0])))
    if key not in ctx.shared:
        ctx.shared[key] = POSITION_ENCODINGS.get(spec.kind)(spec.params, ctx)
    return ctx.shared[key]


@MIXERS.register("attention")
class Attention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, window (0 = none),
    qkv_bias, out_bias, scale (optional), position (PartSpec or None)."""

    graph_safe = True
    # portions of at least 16 rows go to the tensor-core attention in tiles of 128 query rows, the rest row by row
    NEEDS = StepNeeds(tile_rows=128, tile_min_rows=16)

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        p = params
        self.hidden = int(p["hidden_size"])
        self.nq, self.nkv, self.hd = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        if self.nq % self.nkv:
            raise ConfigError("num_heads must be a multiple of num_kv_heads")
        if self.hd % 16 or self.hd > 256:
            raise ConfigError(f"head_dim {self.hd} is not supported (multiples of 16 up to 256)")
        self.window = int(p.get("window", 0) or 0)
        self.qkv_bias = bool(p.get("qkv_bias", False))
        self.out_bias = bool(p.get("out_bias", False))
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.hd)
        self.position = shared_position_encoding(p["position"], ctx) if p.get("position") is not None else None
        self.rot = self.position.rotary_dim if self.position is not None else 0
        self.rot_style = self.position.style if self.position is not None else "half"
        if self.rot > self.hd:
            raise ConfigError("rotary_dim exceeds head_dim")

    def weights(self):
        nq, nkv, hd, H = self.nq, self.nkv, self.hd, self.hidden
        w = {"q_proj.weight": mat(nq * hd, H), "k_proj.weight": mat(nkv * hd, H),
             "v_proj.weight": mat(nkv * hd, H), "o_proj.weight": mat(H, nq * hd)}
        if self.qkv_bias:
            w.update({"q_proj.bias": vec(nq * hd), "k_proj.bias": vec(nkv * hd), "v_proj.bias": vec(nkv * hd)})
        if self.out_bias:
            w["o_proj.bias"] = vec(H)
        return w

    def fused(self):
        f = {"qkv_proj.weight": ["q_proj.weight", "k_proj.weight", "v_proj.weight"]}
        if self.qkv_bias:
            f["qkv_proj.bias"] = ["q_proj.bias", "k_proj.bias", "v_proj.bias"]
        return f

    def load(self, t):
        dt = matmul_dtype(t["q_proj.weight"], t["k_proj.weight"], t["v_proj.weight"])
        self.w_qkv = torch.cat([t["q_proj.weight"].to(dt), t["k_proj.weight"].to(dt), t["v_proj.weight"].to(dt)], 0)
        self.b_qkv = (torch.cat([t["q_proj.bias"], t["k_proj.bias"], t["v_proj.bias"]], 0).contiguous()
                      if self.qkv_bias else None)
        self.w_o = t["o_proj.weight"]
        self.b_o = t.get("o_proj.bias")
        if self.position is not None:
            self.cos, self.sin = self.position.tables()
        else:
            self.cos = self.sin = torch.zeros((1, 1), dtype=torch.float32, device=self.ctx.device)

    def input_dtypes(self):
        return (self.w_qkv.dtype,)

    def cache_spec(self):
        return KVSpec(self.nkv, self.hd, self.window)

    def step_needs(self):
        return self.NEEDS

    def plan_step(self, step, captured):
        """How the key ranges of a batch of decoded tokens are cut.  Requests of about the same length share one
        way of cutting their keys; a ragged batch lets the kernel cut the keys of all rows into equal runs
        itself.  In a captured step the splits are chosen for a bucketed context length, so that few graphs are
        needed as requests grow: four buckets per doubling of the context, at least 256 apart."""
        if step.n_tokens != len(step.entries):
            return None
        lens = [e.start_pos + 1 for e in step.entries]
        step.even_lengths = min(lens) * 4 >= max(lens) * 3
        if not captured:
            return (step.even_lengths,)
        kv = max(step.max_kv_len, 1)
        gran = max(256, 1 << max(kv.bit_length() - 3, 0))
        step.max_kv_len = -(-kv // gran) * gran
        return (step.max_kv_len, step.even_lengths)

    def forward(self, x, residual, step, cache, state, writes_cache=True):
        if cache is None:
            raise ModelError("attention needs a cache")
        ops, nq, nkv, hd = self.ops, self.nq, self.nkv, self.hd
        xin = x[self.w_qkv.dtype]
        T = xin.shape[0]
        act = self.ctx.act_dtype
        q = torch.empty((T, nq * hd), dtype=act, device=xin.device)
        fused = None
        if writes_cache:
            # the projection is left as partial sums over pieces of K; the rotary kernel adds them and the bias
            qkv = ops.gemm_partials(xin, self.w_qkv)
            if T == len(step.entries) and hasattr(ops, "rope_attention_decode"):
                # decoded tokens: one kernel rotates, writes the cache pages and attends
                attn = torch.empty_like(q)
                if ops.rope_attention_decode(qkv, self.b_qkv, self.cos, self.sin, self.rot, self.rot_style, cache, step,
                                             attn, nq, nkv, hd, self.window, self.scale):
                    fused = attn
        if fused is not None:
            attn = fused
        elif writes_cache:
            ops.rope_kv_write(qkv, step.pos, step.slot, self.cos, self.sin, self.rot, q, cache, nq, nkv, hd,
                              True, step.status, bias=self.b_qkv, style=self.rot_style)
        else:   # reads another call's cache: only the queries are needed
            width, nqd = (nq + 2 * nkv) * hd, nq * hd
            qkv = torch.empty((1, T, width), dtype=torch.float32, device=xin.device)
            ops.gemm(xin, self.w_qkv[:nqd], qkv[0, :, :nqd], bias=self.b_qkv[:nqd] if self.b_qkv is not None else None)
            ops.rope_kv_write(qkv, step.pos, step.slot, self.cos, self.sin, self.rot, q, cache, nq, nkv, hd,
                              False, step.status, style=self.rot_style)
        if fused is None:
            attn = torch.empty_like(q)
            ops.attention(q, cache, step, attn, nq, nkv, hd, self.window, self.scale, tiling=step.tiling(self.NEEDS))
        # the output projection is handed to the next norm as partial sums (and its bias)
        return Pending(partials=ops.gemm_partials(attn, self.w_o), bias=self.b_o)
