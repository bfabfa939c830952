"""The description a model is built from: parts chosen layer by layer, and the order
in which layers run, all as data.

An architecture turns its typed configuration into one ``ModelSpec``; the generic
model (``flint_b200.engine.model``) builds parts from it through the registries and
never looks at the architecture's name again.  The reference describes per-layer
variation with per-layer vectors on one config struct (``windows[]``, ``head_dims[]``,
``layer_rope[]``, ``kv_shared``: crates/thuban_architectures/src/transformer/config.rs:30-58);
here each layer carries its own part specs instead.
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class PartSpec:
    """A part by registry name with its sizes and constants."""
    kind: str
    params: dict = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (``block``) of parts by role, and where each role's
    tensors live under the layer's prefix (``names[role]`` -> sub-prefix)."""
    block: str
    parts: dict            # role -> PartSpec, e.g. norm1 / mixer / norm2 / ffn
    prefix: str            # e.g. "layers.3."
    names: dict            # role -> tensor sub-prefix, e.g. {"mixer": "self_attn."}


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.  ``layer`` indexes ``ModelSpec.layers`` (a layer may
    be called more than once: its weights are shared, each call has a cache of its
    own).  ``cache_of`` names an earlier entry of the order whose cache this call
    reads instead of writing one of its own."""
    layer: int
    cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    layers: tuple            # of LayerSpec
    order: tuple             # of LayerCall
    final_norm: PartSpec
    embed_name: str = "embed_tokens."
    final_norm_name: str = "norm."
    head_name: str = "lm_head."
    head_bias: bool = False
    tie_word_embeddings: bool = False
    embed_scale: float = 1.0
    eos_token_ids: tuple = ()
    # A position encoding that acts on the embedded rows instead of inside a mixer (learned absolute positions
    # and the like): a PartSpec of the position-encoding registry whose part has ``after_embedding(h, step)``;
    # its tensors live under ``embed_position_name``.
    embed_position: PartSpec | None = None
    embed_position_name: str = "embed_positions."
