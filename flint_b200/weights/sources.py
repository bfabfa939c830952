"""Where tensors come from: a folder of safetensors files, or a seeded random source.

Both answer ``names()`` and ``read(name, spec, device)``.  The reference has the same
pair behind one trait: a memory-mapped checkpoint reader and a synthetic checkpoint
for its benchmark (crates/thuban_checkpoint/src/lib.rs:145-149,
crates/thuban_bench/src/synth.rs:96-156).
"""
from __future__ import annotations

import json
import zlib
from dataclasses import dataclass
from pathlib import Path

import torch

from ..errors import WeightError
from .safetensors_io import SafetensorsFile


@dataclass(frozen=True)
class WeightSpec:
    """What a part expects of one tensor.

    role: ``"matrix"`` (kept in the stored floating type: bfloat16 stays bfloat16, a
    tensor stored in 32-bit stays 32-bit; everything is 32-bit in the float32 mode),
    ``"vector"`` (norm scales and biases: widened to float32, which is exact), or
    ``"table"`` (integer table, kept as int32).
    init: how the random source fills it: ``"normal"`` N(0, std), ``"gamma"`` 1+N(0, 0.1).
    """
    shape: tuple
    role: str = "matrix"
    init: str = "normal"
    std: float = 0.02
    optional: bool = False


class SafetensorsSource:
    """``model.safetensors`` in a folder, or the shards named by
    ``model.safetensors.index.json``.  A leading ``model.`` is dropped from names."""

    def __init__(self, model_dir):
        self.dir = Path(model_dir)
        index = self.dir / "model.safetensors.index.json"
        single = self.dir / "model.safetensors"
        files = []
        if single.is_file():
            files = [single]
        elif index.is_file():
            wm = json.loads(index.read_text()).get("weight_map", {})
            files = sorted({self.dir / f for f in wm.values()})
        else:
            raise WeightError(f"{self.dir}: neither model.safetensors nor model.safetensors.index.json found")
        self._files = [SafetensorsFile(f) for f in files]
        self._where = {}
        for f in self._files:
            for raw in f.names():
                name = raw[len("model."):] if raw.startswith("model.") else raw
                if name in self._where:
                    raise WeightError(f"tensor {name!r} appears twice in {self.dir}")
                self._where[name] = (f, raw)

    def names(self):
        return list(self._where)

    def shape(self, name):
        f, raw = self._where[name]
        return f.shape(raw)

    def dtype(self, name):
        f, raw = self._where[name]
        return f.dtype(raw)

    def read(self, name, spec: WeightSpec | None = None, device="cpu") -> torch.Tensor:
        f, raw = self._where[name]
        return f.read(raw).to(device)

    def close(self):
        for f in self._files:
            f.close()


class RandomSource:
    """Seeded random tensors for a given set of specs.  Every tensor has its own
    generator seeded by (seed, crc32(name)), so one tensor's values do not depend on
    which others are drawn or in what order."""

    def __init__(self, specs: dict, seed: int, dtype=torch.bfloat16, on_device=False):
        self.specs = dict(specs)
        self.seed = int(seed)
        self.store_dtype = dtype
        self.on_device = on_device

    def names(self):
        return [n for n, s in self.specs.items()]

    def shape(self, name):
        return tuple(self.specs[name].shape)

    def dtype(self, name):
        s = self.specs[name]
        return torch.int32 if s.role == "table" else self.store_dtype

    def read(self, name, spec: WeightSpec | None = None, device="cpu") -> torch.Tensor:
        spec = self.specs[name]
        gen_dev = device if (self.on_device and str(device) != "cpu") else "cpu"
        g = torch.Generator(device=gen_dev)
        g.manual_seed((self.seed * 0x9E3779B1 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFFFFFF)
        if spec.role == "table":
            return torch.randint(0, 2 ** 15, spec.shape, generator=g, device=gen_dev, dtype=torch.int32).to(device)
        if gen_dev == "cpu":
            t = torch.randn(spec.shape, generator=g, dtype=torch.float32)
        else:
            # large models: draw on the device in the stored type, piecewise, to bound the peak
            t = torch.empty(spec.shape, device=gen_dev, dtype=self.store_dtype)
            t.normal_(0.0, 1.0, generator=g)
        if spec.init == "gamma":
            t = t.mul_(0.1).add_(1.0)
        else:
            t = t.mul_(spec.std)
        return t.to(self.store_dtype).to(device)
