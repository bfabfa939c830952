"""Matching a source's tensors against what the model expects, with one clear error.

The reference fails on the first missing tensor
(crates/thuban_model/src/loader.rs:23-27); here every fault is collected first so that
one message lists all missing names, all unexpected names and all wrong shapes.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..errors import WeightError
from .safetensors_io import save_safetensors
from .sources import FusedView, RandomSource, WeightSpec


def check_names_and_shapes(source, expected: dict):
    """Raise one WeightError listing every mismatch between ``source`` and ``expected``
    (name -> WeightSpec)."""
    have = set(source.names())
    missing = sorted(n for n, s in expected.items() if n not in have and not s.optional)
    unexpected = sorted(have - set(expected))
    wrong = []
    for n, s in expected.items():
        if n in have and tuple(source.shape(n)) != tuple(s.shape):
            wrong.append(f"{n}: expected {tuple(s.shape)}, found {tuple(source.shape(n))}")
        elif n in have:
            dt = source.dtype(n)
            if s.role == "table" and dt.is_floating_point or s.role != "table" and not dt.is_floating_point:
                wrong.append(f"{n}: expected {'an integer' if s.role == 'table' else 'a floating'} type, found {dt}")
    wrong += list(getattr(source, "problems", ()))
    if missing or unexpected or wrong:
        lines = ["checkpoint does not match the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes or types ({len(wrong)}): " + "; ".join(wrong))
        raise WeightError("\n".join(lines))


def place(t: torch.Tensor, spec: WeightSpec, compute: str, device) -> torch.Tensor:
    """Type policy.  float32 mode: every floating tensor becomes float32.  bfloat16
    mode: matrices stay as stored when stored as bfloat16 or float32 (other floating
    types become bfloat16); vectors become float32; integer tables become int32."""
    if spec.role == "table":
        return t.to(device=device, dtype=torch.int32).contiguous()
    if compute == "float32" or spec.role == "vector":
        return t.to(device=device, dtype=torch.float32).contiguous()
    if t.dtype in (torch.bfloat16, torch.float32):
        return t.to(device=device).contiguous()
    return t.to(device=device, dtype=torch.bfloat16).contiguous()


def load_tensors(source, expected: dict, compute: str, device, fused: dict | None = None) -> dict:
    """All expected tensors, checked, converted by ``place`` and moved to ``device``.  ``fused``: fused tensor
    name -> the expected tensors it may stand for, stacked by rows (see ``FusedView``)."""
    if fused:
        source = FusedView(source, fused, expected)
    check_names_and_shapes(source, expected)
    out = {}
    have = set(source.names())
    for name, spec in expected.items():
        if name not in have:
            continue
        out[name] = place(source.read(name, spec, device), spec, compute, device)
    return out


def write_model_folder(out_dir, config_dict: dict, expected: dict, seed: int,
                       dtype=torch.bfloat16, name_prefix="model.", head_prefix="lm_head."):
    """Random-weights mode: write ``config.json`` and ``model.safetensors`` for a
    configuration and a seed.  Names get the customary ``model.`` prefix, except the
    output head."""
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    (out_dir / "config.json").write_text(json.dumps(config_dict, indent=1))
    src = RandomSource(expected, seed, dtype=dtype)

    class _Lazy:
        def __init__(self, name):
            self.name = name
            self.shape = tuple(expected[name].shape)
            self.dtype = src.dtype(name)

        def __call__(self):
            return src.read(self.name)

    tensors = {}
    for name in expected:
        stored = name if name.startswith(head_prefix) else name_prefix + name
        tensors[stored] = _Lazy(name)
    save_safetensors(out_dir / "model.safetensors", tensors, metadata={"format": "pt", "seed": seed})
    return out_dir
