"""Sampling options with the reference's names, defaults and meanings
(crates/thuban_generate/src/sampler.rs:8-35)."""
from __future__ import annotations

from dataclasses import dataclass

M64 = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.7     # <= 0: greedy
    top_k: int = 20              # 0: off
    top_p: float = 0.8           # >= 1: off
    min_p: float = 0.0           # relative floor against the largest probability
    repeat_penalty: float = 1.0  # 1: off
    repeat_last_n: int = 64      # how many of the generated tokens are penalised

    @classmethod
    def greedy(cls):
        return cls(temperature=0.0)


class SplitMix64:
    """The reference's generator: one splitmix64 step per draw, u = (z >> 40) / 2^24
    (crates/thuban_generate/src/sampler.rs:135-142)."""

    def __init__(self, seed: int):
        self.state = int(seed) & M64

    def next_f32(self) -> float:
        self.state = (self.state + 0x9E3779B97F4A7C15) & M64
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
        z ^= z >> 31
        return (z >> 40) / float(1 << 24)
