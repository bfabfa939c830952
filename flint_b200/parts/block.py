"""Arrangements of a layer's parts.

``prenorm``: h += mixer(norm1(h)); h += ffn(norm2(h)) -- the reference's decoder layer
(crates/thuban_architectures/src/transformer/forward.rs:102-440) and Phi-MoE's.
``parallel``: h += mixer(norm1(h)) + ffn(norm1(h)) with one shared norm.
An arrangement only orders parts; it does not know what they are.
"""
from __future__ import annotations

from ..registry import BLOCKS


class Block:
    roles = ()

    def __init__(self, parts: dict):
        self.parts = parts

    def forward(self, residual, step, cache, state, writes_cache=True):
        raise NotImplementedError


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    roles = ("norm1", "mixer", "norm2", "ffn")

    def forward(self, residual, step, cache, state, writes_cache=True):
        p = self.parts
        x = p["norm1"].forward(residual, p["mixer"].input_dtypes())
        p["mixer"].forward(x, residual, step, cache, state, writes_cache)
        x = p["norm2"].forward(residual, p["ffn"].input_dtypes())
        p["ffn"].forward(x, residual, step)


@BLOCKS.register("parallel")
class ParallelBlock(Block):
    roles = ("norm1", "mixer", "ffn")

    def forward(self, residual, step, cache, state, writes_cache=True):
        p = self.parts
        want = tuple(set(p["mixer"].input_dtypes()) | set(p["ffn"].input_dtypes()))
        x = p["norm1"].forward(residual, want)
        p["mixer"].forward(x, residual, step, cache, state, writes_cache)
        p["ffn"].forward(x, residual, step)
