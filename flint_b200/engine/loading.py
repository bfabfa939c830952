"""Entry points for getting a model: from a folder, or written from a configuration and a seed."""
from __future__ import annotations

import torch

from ..parts.base import BuildContext
from ..weights.loader import write_model_folder
from ..weights.sources import WeightSpec
from .model import Layer, Model, architecture_of, load_model  # noqa: F401


def expected_from_config(config: dict):
    """(spec, {tensor name: WeightSpec}) for a config.json dictionary, without a device."""
    from .. import models  # noqa: F401
    from ..registry import NORMS
    arch = architecture_of(config)
    spec = arch.model_spec(arch.parse_config(config))
    ctx = BuildContext(ops=None, device=torch.device("cpu"), compute="float32")
    expected = {spec.embed_name + "weight": WeightSpec((spec.vocab_size, spec.hidden_size))}
    for ls in spec.layers:
        expected.update(Layer(ls, ctx).weights())
    fn = NORMS.get(spec.final_norm.kind)(spec.final_norm.params, ctx)
    for name, ws in fn.weights().items():
        expected[spec.final_norm_name + name] = ws
    if not spec.tie_word_embeddings:
        expected[spec.head_name + "weight"] = WeightSpec((spec.vocab_size, spec.hidden_size))
    if spec.head_bias:
        expected[spec.head_name + "bias"] = WeightSpec((spec.vocab_size,), role="vector")
    return spec, expected


def write_random_model(out_dir, config: dict, seed: int = 0, dtype=torch.bfloat16):
    """Random-weights mode: write ``config.json`` and ``model.safetensors`` for a
    configuration and a seed (weights and biases N(0, 0.02), norm scales 1 + N(0, 0.1))."""
    _, expected = expected_from_config(config)
    return write_model_folder(out_dir, config, expected, seed, dtype=dtype)
