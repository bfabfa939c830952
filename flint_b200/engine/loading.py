"""Entry points for getting a model: from a folder, or written from a configuration and a seed."""
from __future__ import annotations

import torch

from ..parts.base import BuildContext
from ..weights.loader import write_model_folder
from ..weights.sources import RandomSource, WeightSpec
from .model import Layer, Model, architecture_of, expected_tensors, fused_tensors, load_model  # noqa: F401


def expected_from_config(config: dict, with_fused=False):
    """(spec, {tensor name: WeightSpec}) for a config.json dictionary, without a device; with ``with_fused``
    also the fused tensors a checkpoint may store instead (fused name -> names it stands for)."""
    from .. import models  # noqa: F401
    from ..registry import NORMS
    arch = architecture_of(config)
    spec = arch.model_spec(arch.parse_config(config))
    ctx = BuildContext(ops=None, device=torch.device("cpu"), compute="float32")
    layers = [Layer(ls, ctx) for ls in spec.layers]
    from ..registry import POSITION_ENCODINGS
    embed_position = (POSITION_ENCODINGS.get(spec.embed_position.kind)(spec.embed_position.params, ctx)
                      if spec.embed_position is not None else None)
    expected = expected_tensors(spec, layers, NORMS.get(spec.final_norm.kind)(spec.final_norm.params, ctx), embed_position)
    return (spec, expected, fused_tensors(layers)) if with_fused else (spec, expected)


def write_random_model(out_dir, config: dict, seed: int = 0, dtype=torch.bfloat16):
    """Random-weights mode: write ``config.json`` and ``model.safetensors`` for a
    configuration and a seed (weights and biases N(0, 0.02), norm scales 1 + N(0, 0.1))."""
    _, expected = expected_from_config(config)
    return write_model_folder(out_dir, config, expected, seed, dtype=dtype)


def random_model(config: dict, seed: int = 0, *, dtype="bfloat16", store_dtype=None, on_device=False, **model_kw) -> Model:
    """Random-weights mode without a folder: the model that ``config`` (a config.json dictionary) names, with the
    tensors that ``write_random_model`` would write for the same seed and stored type (default: the compute
    type), drawn straight into the model.  ``on_device`` draws large models on the GPU (other values)."""
    spec, expected = expected_from_config(config)
    if store_dtype is None:
        store_dtype = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    return Model(spec, RandomSource(expected, seed, dtype=store_dtype, on_device=on_device), dtype=dtype, **model_kw)
