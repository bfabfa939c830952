"""What every part of a layer looks like to the model that holds it.

A part gets its sizes and constants as parameters, names the tensors it expects under
its own prefix, receives them once, and then runs on whatever rows a step brings.
No part knows which architecture it is in; the reference's ops take spec structs in
the same spirit (``NormSpec``, ``AttnSpec``, ``RopeArgs``, ``MlpSpec``:
crates/thuban_model/src/ops/*.rs).

Interfaces
----------
Norm          ``forward(x, want, row_index=None, pending=None, router=None) -> {dtype: tensor}``
              x is the float32 residual stream [T, H]; ``want`` is the set of element
              types the next part asked for.  A norm with ``supports_pending`` applies a
              ``Pending`` addition to x first; one with ``supports_router`` can fill a
              ``RouterRequest``.  Both are optional abilities; the block works without them.
Mixer         ``input_dtypes()``, ``cache_spec()``, ``state_spec()``, optionally ``step_needs()`` (rows cut into
              tiles) and ``plan_step(step, captured)`` (how this step's work is cut),
              ``forward(x, residual, step, cache, state, writes_cache=True)``:
              adds its output into ``residual`` (float32 [T, H]) in place and returns None,
              or returns a ``Pending`` that the block hands to the next norm.
FeedForward   ``input_dtypes()``, ``forward(x, residual, step)``: adds into ``residual`` or
              returns a ``Pending``.  A feed-forward with ``router_request(n_rows)`` gets the
              filled request back as ``forward(..., routed=request)``.
PositionEncoding  ``rotary_dim``, ``style`` ("half": dims i and i + rotary_dim/2 rotate together, "interleaved":
              dims 2i and 2i + 1), ``tables() -> (cos, sin)`` float32 [positions, rotary_dim/2]; one named by
              ``ModelSpec.embed_position`` instead has ``after_embedding(h, step)`` and adds to the embedded rows.
Block         ``forward(residual, step, cache, state, writes_cache)``: the arrangement of
              the parts of one layer.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..weights.sources import WeightSpec


@dataclass
class Pending:
    """An addition to the residual stream that its producer has not applied: the next norm's
    kernel applies it while it reads the row anyway (or ``ops.apply_pending`` does, for a norm
    that cannot).  Either partial sums of a product whose K range was split
    (``partials`` [S, T, H] float32, plus an optional ``bias`` [H]), or the two selected experts'
    outputs (``y`` [2T, H] with ``row_of`` [T, 2] and ``gates`` [T, 2]), or both."""
    partials: torch.Tensor | None = None
    bias: torch.Tensor | None = None
    y: torch.Tensor | None = None
    row_of: torch.Tensor | None = None
    gates: torch.Tensor | None = None


@dataclass
class RouterRequest:
    """What a feed-forward asks a norm to compute while the normalised row is at hand: router
    logits over ``weight`` [E, H], sparsemixer top-2 with ``jitter_eps``, into ``expert_ids`` and
    ``gates`` ([T, 2] each).  ``logits`` ([T, E] float32, optional): the logits the choice was made from
    are written there too (tests compare them)."""
    weight: torch.Tensor
    jitter_eps: float
    expert_ids: torch.Tensor
    gates: torch.Tensor
    logits: torch.Tensor | None = None


@dataclass
class BuildContext:
    """What parts need to know about where they run."""
    ops: object                    # the kernel set
    device: torch.device
    compute: str                   # "bfloat16" or "float32"
    shared: dict = field(default_factory=dict)   # things built once per model (position tables)

    @property
    def act_dtype(self):
        return torch.bfloat16 if self.compute == "bfloat16" else torch.float32


class Part:
    """Base of all parts: parameters in, tensor specs out, tensors in."""

    # True if ``forward`` only launches work that reads the step's metadata from device memory
    # (so a decode step can be captured once as a CUDA graph and replayed).  A part that looks at
    # the host-side entries of the step must leave this False; the model then runs it eagerly.
    graph_safe = False

    def __init__(self, params: dict, ctx: BuildContext):
        self.params = dict(params)
        self.ctx = ctx
        self.ops = ctx.ops

    def weights(self) -> dict:
        """name (under this part's prefix) -> WeightSpec"""
        return {}

    def fused(self) -> dict:
        """Fused tensors a checkpoint may store instead of some of ``weights()``: fused name -> the names it
        stands for, stacked by rows in that order (all under this part's prefix)."""
        return {}

    def load(self, tensors: dict):
        """Receives the tensors named by ``weights()`` (already on the device and typed
        by the loader's policy)."""

    def input_dtypes(self):
        return (self.ctx.act_dtype,)


class Mixer(Part):
    def cache_spec(self):
        return None

    def state_spec(self):
        return None

    def step_needs(self):
        """A ``StepNeeds`` if the mixer wants the step's rows cut into tiles (see ``engine/step.py``), else None."""
        return None

    def plan_step(self, step, captured: bool):
        """Called once per step (on one mixer of each kind) before the layers run, with the host-side view of
        the batch: the mixer may work out how it will cut its work (into ``step.plans[kind]`` or the fields it
        reads later) and returns a hashable value naming everything about the plan that shapes its launches,
        or None.  A decode step that is captured as a CUDA graph (``captured``) is keyed by these values, so a
        graph is only replayed on steps that would launch the same work."""
        return None

    def forward(self, x, residual, step, cache, state, writes_cache=True):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, residual, step):
        raise NotImplementedError


class Norm(Part):
    supports_pending = False
    supports_router = False

    def forward(self, x, want, row_index=None, pending=None, router=None):
        raise NotImplementedError


class PositionEncoding(Part):
    rotary_dim = 0
    style = "half"          # which dims of a head rotate together: "half" (i, i + rotary_dim/2) or "interleaved" (2i, 2i + 1)

    def tables(self):
        raise NotImplementedError


def matmul_dtype(*ws):
    """The element type a product over these stored matrices runs in: bfloat16 only if
    all of them are bfloat16, else float32."""
    return torch.bfloat16 if all(w.dtype == torch.bfloat16 for w in ws) else torch.float32


def vec(n, init="normal", optional=False):
    return WeightSpec((n,), role="vector", init=init, optional=optional)


def mat(*shape):
    return WeightSpec(tuple(shape), role="matrix")
