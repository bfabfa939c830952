"""Arrangements of a layer's parts.

``prenorm``: h += mixer(norm1(h)); h += ffn(norm2(h)) -- the reference's decoder layer
(crates/thuban_architectures/src/transformer/forward.rs:102-440) and Phi-MoE's.
``parallel``: h += mixer(norm1(h)) + ffn(norm1(h)) with one shared norm.
An arrangement only orders parts; it does not know what they are.
"""
from __future__ import annotations

import torch

from ..registry import BLOCKS


def run_norm(norm, residual, want, pending=None, router=None, row_index=None):
    """Run a norm; a pending addition or a routing request that the norm cannot take is served
    by separate kernels instead.  Returns (outputs, router or None if it still has to be done)."""
    if pending is not None and not norm.supports_pending:
        norm.ops.apply_pending(residual, pending)
        pending = None
    if router is not None and not norm.supports_router:
        router = None
    kw = {}
    if pending is not None:
        kw["pending"] = pending
    if router is not None:
        kw["router"] = router
    if row_index is not None:
        kw["row_index"] = row_index
    return norm.forward(residual, want, **kw), router


def settle(part, residual, pending):
    """Apply a pending addition right away (for arrangements that cannot carry it)."""
    if pending is not None:
        part.ops.apply_pending(residual, pending)


class Block:
    roles = ()

    def __init__(self, parts: dict):
        self.parts = parts

    def forward(self, residual, step, cache, state, writes_cache=True, carry=None):
        """Runs the layer on ``residual`` in place.  ``carry``: a Pending addition left by the
        previous layer; returns the Pending addition this layer leaves (or None)."""
        raise NotImplementedError


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    roles = ("norm1", "mixer", "norm2", "ffn")

    def forward(self, residual, step, cache, state, writes_cache=True, carry=None):
        p = self.parts
        mixer, ffn = p["mixer"], p["ffn"]
        x, _ = run_norm(p["norm1"], residual, mixer.input_dtypes(), carry)
        pend = mixer.forward(x, residual, step, cache, state, writes_cache)
        request = ffn.router_request(residual.shape[0]) if hasattr(ffn, "router_request") else None
        if request is not None and step.record is not None and getattr(request, "logits", 0) is None:
            # a test asked for this step's internals: the logits behind the routing come along
            request.logits = request.weight.new_empty((residual.shape[0], request.weight.shape[0]), dtype=torch.float32)
        want = ffn.input_dtypes_when_routed() if request is not None and p["norm2"].supports_router \
            else ffn.input_dtypes()
        x, routed = run_norm(p["norm2"], residual, want, pend, request)
        return ffn.forward(x, residual, step, routed=routed) if routed is not None else ffn.forward(x, residual, step)


@BLOCKS.register("parallel")
class ParallelBlock(Block):
    roles = ("norm1", "mixer", "ffn")

    def forward(self, residual, step, cache, state, writes_cache=True, carry=None):
        p = self.parts
        want = tuple(set(p["mixer"].input_dtypes()) | set(p["ffn"].input_dtypes()))
        x, _ = run_norm(p["norm1"], residual, want, carry)
        settle(p["mixer"], residual, p["mixer"].forward(x, residual, step, cache, state, writes_cache))
        return p["ffn"].forward(x, residual, step)
