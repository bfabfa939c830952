"""Rotary position encoding with optional LongRoPE scaling.

The cos/sin tables are built on the host in float64 and stored as float32
[positions, rotary_dim/2]: inv_i = theta^(-2i/rot), divided by the short factor for
positions below the original context length and by the long factor from there on.
The choice is made per position, as the reference does
(crates/thuban_model/src/ops/rope.rs:52-87), so a cached key never has to be rotated
again and the logits do not depend on how a prompt was cut.  The LongRoPE magnitude
scale (short_mscale / long_mscale, again per position) multiplies cos and sin; the
reference has no such scale.  The rotation itself (NeoX half-split) is done by the
kernel that also writes keys and values into the cache.
"""
from __future__ import annotations

import torch

from ..errors import ConfigError
from ..registry import POSITION_ENCODINGS
from .base import PositionEncoding


@POSITION_ENCODINGS.register("rope")
class RotaryEncoding(PositionEncoding):
    """params: rotary_dim, theta, max_positions, and for LongRoPE: short_factor,
    long_factor, original_max_positions, short_mscale, long_mscale."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.rotary_dim = int(params["rotary_dim"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ConfigError(f"rotary_dim must be even and positive, got {self.rotary_dim}")
        self.theta = float(params["theta"])
        self.max_positions = int(params["max_positions"])
        self._tables = None

    def tables(self):
        if self._tables is None:
            half = self.rotary_dim // 2
            i = torch.arange(half, dtype=torch.float64)
            inv = self.theta ** (-2.0 * i / self.rotary_dim)
            pos = torch.arange(self.max_positions, dtype=torch.float64)
            p = self.params
            if p.get("short_factor") is not None:
                short = torch.tensor(p["short_factor"], dtype=torch.float64)
                long = torch.tensor(p["long_factor"], dtype=torch.float64)
                if short.numel() != half or long.numel() != half:
                    raise ConfigError(f"LongRoPE factor lists must have {half} entries")
                is_short = (pos < int(p["original_max_positions"]))[:, None]
                ang = pos[:, None] * torch.where(is_short, inv / short, inv / long)
                scale = torch.where(is_short, torch.tensor(float(p.get("short_mscale", 1.0)), dtype=torch.float64),
                                    torch.tensor(float(p.get("long_mscale", 1.0)), dtype=torch.float64))
            else:
                ang = pos[:, None] * inv[None, :]
                scale = torch.ones((1, 1), dtype=torch.float64)
            cos = (torch.cos(ang) * scale).to(torch.float32).contiguous().to(self.ctx.device)
            sin = (torch.sin(ang) * scale).to(torch.float32).contiguous().to(self.ctx.device)
            self._tables = (cos, sin)
        return self._tables
