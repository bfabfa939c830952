"""Builds and runs the C++ plain implementation (tests/plain_phimoe.cpp)."""
from __future__ import annotations

import hashlib
import os
import struct
import subprocess
import tempfile
from pathlib import Path

SOURCE = Path(__file__).with_name("plain_phimoe.cpp")


def build() -> str:
    """Compile with the host compiler (once per source text) and return the program's path."""
    tag = hashlib.sha256(SOURCE.read_bytes()).hexdigest()[:16]
    out_dir = Path(tempfile.gettempdir()) / f"flint_plain_cpp_{os.getuid()}"
    out_dir.mkdir(parents=True, exist_ok=True)
    exe = out_dir / f"plain_phimoe_{tag}"
    if not exe.is_file():
        tmp = exe.with_suffix(f".{os.getpid()}.tmp")
        subprocess.run([os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-o", str(tmp), str(SOURCE)], check=True)
        os.replace(tmp, exe)
    return str(exe)


def logits(model_dir, requests, n_layers, vocab):
    """[(logits [T][V] as a flat list of floats, experts [layers][T][2])] for lists of token ids."""
    exe = build()
    with tempfile.TemporaryDirectory() as d:
        tok = Path(d) / "tokens.txt"
        tok.write_text("".join(" ".join(map(str, r)) + "\n" for r in requests))
        out = Path(d) / "out.bin"
        subprocess.run([exe, "logits", str(model_dir), str(tok), str(out)], check=True)
        raw = out.read_bytes()
    res, o = [], 0
    for r in requests:
        T = len(r)
        lg = struct.unpack_from(f"<{T * vocab}f", raw, o)
        o += 4 * T * vocab
        ex = struct.unpack_from(f"<{n_layers * T * 2}i", raw, o)
        o += 4 * n_layers * T * 2
        res.append((lg, ex))
    assert o == len(raw)
    return res


def generate(model_dir, prompts, n_tokens, temperature=0.0, top_k=0, top_p=1.0, seed=42):
    """(token lists, seconds) of the program's generation, every token from a whole-sequence forward pass."""
    exe = build()
    with tempfile.TemporaryDirectory() as d:
        tok = Path(d) / "prompts.txt"
        tok.write_text("".join(" ".join(map(str, r)) + "\n" for r in prompts))
        proc = subprocess.run([exe, "generate", str(model_dir), str(tok), str(n_tokens), repr(float(temperature)),
                               str(int(top_k)), repr(float(top_p)), str(int(seed))], check=True, capture_output=True, text=True)
    lines = proc.stdout.strip().split("\n")
    secs = float(lines[-1].split()[1])
    return [[int(x) for x in l.split()] for l in lines[:-1]], secs
