"""Reading and writing the safetensors container, by tensor name.

The format is an 8-byte little-endian header length, a JSON header mapping each name
to ``{"dtype", "shape", "data_offsets"}`` and then the raw little-endian tensor
bytes.  The reference reads checkpoints through one trait with ``names()`` and
``read(name)`` over a memory map (crates/thuban_checkpoint/src/lib.rs:145-149); this
is the same interface over safetensors.
"""
from __future__ import annotations

import json
import mmap
import struct
import warnings
from pathlib import Path

import torch

from ..errors import WeightError

_TO_TORCH = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_FROM_TORCH = {v: k for k, v in _TO_TORCH.items()}


class SafetensorsFile:
    """One ``.safetensors`` file, memory-mapped; tensors are read one at a time."""

    def __init__(self, path):
        self.path = Path(path)
        try:
            self._fh = open(self.path, "rb")
        except OSError as e:
            raise WeightError(f"cannot open {self.path}: {e}") from None
        head = self._fh.read(8)
        if len(head) != 8:
            raise WeightError(f"{self.path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", head)
        size = self.path.stat().st_size
        if n <= 0 or 8 + n > size:
            raise WeightError(f"{self.path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._fh.read(n))
        except ValueError as e:
            raise WeightError(f"{self.path}: header is not valid JSON: {e}") from None
        self.metadata = header.pop("__metadata__", {})
        self._info = header
        self._data_start = 8 + n
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else None
        for name, info in header.items():
            if info.get("dtype") not in _TO_TORCH:
                raise WeightError(f"{self.path}: tensor {name!r} has unsupported dtype {info.get('dtype')!r}")
            lo, hi = info["data_offsets"]
            if not (0 <= lo <= hi <= size - self._data_start):
                raise WeightError(f"{self.path}: tensor {name!r} lies outside the file")

    def names(self):
        return list(self._info)

    def shape(self, name):
        return tuple(self._info[name]["shape"])

    def dtype(self, name):
        return _TO_TORCH[self._info[name]["dtype"]]

    def read(self, name) -> torch.Tensor:
        """A CPU tensor that owns its memory (copied out of the map)."""
        info = self._info[name]
        dtype = _TO_TORCH[info["dtype"]]
        shape = tuple(info["shape"])
        lo, hi = info["data_offsets"]
        count = 1
        for s in shape:
            count *= s
        if count * torch.empty(0, dtype=dtype).element_size() != hi - lo:
            raise WeightError(f"{self.path}: tensor {name!r}: {hi - lo} bytes do not match shape {shape}")
        if count == 0:
            return torch.empty(shape, dtype=dtype)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)   # the read-only map is copied right away
            view = torch.frombuffer(self._mm, dtype=dtype, count=count, offset=self._data_start + lo)
        return view.reshape(shape).clone()

    def close(self):
        if self._mm is not None:
            self._mm.close()
            self._mm = None
        self._fh.close()


def save_safetensors(path, tensors, metadata=None):
    """Write ``tensors`` (name -> CPU tensor, or a callable returning one, so that
    large models need not be held in memory whole) to ``path``."""
    items = []
    offset = 0
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    shapes = {}
    for name, t in tensors.items():
        if callable(t):
            shape, dtype = t.shape, t.dtype
        else:
            shape, dtype = tuple(t.shape), t.dtype
        if dtype not in _FROM_TORCH:
            raise WeightError(f"tensor {name!r}: dtype {dtype} cannot be stored")
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        header[name] = {"dtype": _FROM_TORCH[dtype], "shape": list(shape),
                        "data_offsets": [offset, offset + nbytes]}
        shapes[name] = (shape, dtype, nbytes)
        offset += nbytes
        items.append(name)
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in items:
            t = tensors[name]
            if callable(t):
                t = t()
            t = t.detach().cpu().contiguous()
            shape, dtype, nbytes = shapes[name]
            assert tuple(t.shape) == tuple(shape) and t.dtype == dtype, name
            if nbytes:
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else
                        t.reshape(1).view(torch.uint8).numpy().tobytes())
