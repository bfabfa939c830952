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


class FusedView:
    """A source seen through the fused tensors it may hold: where a checkpoint stores several of a part's
    matrices stacked by rows in one tensor (q|k|v as ``qkv_proj``, gate|up as ``gate_up_proj``), the pieces
    appear under their own names, each a run of the fused tensor's rows.  The reference splits the same way at
    load (crates/thuban_architectures/src/phi.rs:109-160).

    ``fused``: fused name -> list of piece names, in row order; the row counts come from ``expected``.
    A fused tensor whose shape is not the pieces' rows stacked is reported in ``problems`` (and its pieces stay
    missing), for the loader's one error message."""

    def __init__(self, source, fused: dict, expected: dict):
        self.source = source
        self.problems = []
        self._piece = {}                     # piece name -> (fused name, first row, rows)
        self._hidden = set()                 # fused names that are served as pieces
        have = set(source.names())
        for fname, pieces in fused.items():
            if fname not in have or any(p in have for p in pieces) or any(p not in expected for p in pieces):
                continue                     # absent, or stored both ways (then the fused one is unexpected)
            rows = [int(expected[p].shape[0]) for p in pieces]
            rest = tuple(expected[pieces[0]].shape[1:])
            want = (sum(rows), *rest)
            found = tuple(source.shape(fname))
            self._hidden.add(fname)
            if found != want or any(tuple(expected[p].shape[1:]) != rest for p in pieces):
                self.problems.append(f"{fname}: expected {want} (rows of {' | '.join(pieces)} = "
                                     f"{' + '.join(map(str, rows))}), found {found}")
                continue
            r0 = 0
            for p, n in zip(pieces, rows):
                self._piece[p] = (fname, r0, n)
                r0 += n
        self._cache = (None, None)

    def names(self):
        return [n for n in self.source.names() if n not in self._hidden] + list(self._piece)

    def shape(self, name):
        if name in self._piece:
            fname, _, n = self._piece[name]
            return (n, *tuple(self.source.shape(fname))[1:])
        return self.source.shape(name)

    def dtype(self, name):
        return self.source.dtype(self._piece[name][0] if name in self._piece else name)

    def read(self, name, spec=None, device="cpu"):
        if name not in self._piece:
            return self.source.read(name, spec, device)
        fname, r0, n = self._piece[name]
        if self._cache[0] != fname:          # the pieces of one fused tensor are read one after the other
            self._cache = (fname, self.source.read(fname, None, device))
        return self._cache[1][r0:r0 + n].contiguous()
