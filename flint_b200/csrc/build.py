"""Compiling the CUDA sources of this folder for sm_100a and loading them.

Each ``.cu`` file is one module: it is compiled with nvcc into a shared library of
its own the first time one of its functions is needed, and loaded with ctypes.  The
libraries live next to the sources in ``_build/`` (named by a hash of the sources and
flags, so an edited file is rebuilt), or, if that folder cannot be written, in a
per-user folder under the system's temporary directory.  Nothing needs the network,
a home directory or a pre-built cache.  While a module compiles, a line is printed
to stderr when it starts, every few seconds, and when it ends.

The host runtime (``host/runtime.cpp``: page pools, scheduler, step packing; no device
code) is built the same way with the host C++ compiler.

There is no fallback: if a compiler is missing or a module fails to compile or load, a
``KernelError`` says so.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

from ..errors import KernelError

SRC_DIR = Path(__file__).resolve().parent
MODULES = ("elementwise", "row_fused", "gemm_simt", "gemm_tc", "attention", "attention_tc", "moe", "sampling", "noalloc")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC"]
HOST_MODULES = ("runtime",)
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC"]
_LOCK = threading.Lock()
_LOADED: dict[str, ctypes.CDLL] = {}


def available_modules():
    return [m for m in MODULES if (SRC_DIR / f"{m}.cu").is_file()] + \
           [m for m in HOST_MODULES if (SRC_DIR / "host" / f"{m}.cpp").is_file()]


def _nvcc() -> str:
    for cand in (os.environ.get("FLINT_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise KernelError("nvcc not found (looked at $FLINT_NVCC, PATH and /usr/local/cuda/bin); "
                      "the CUDA kernels cannot be built and there is no fallback")


def _host_compiler() -> str:
    for cand in (os.environ.get("FLINT_CXX"), os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"),
                 shutil.which("clang++")):
        if cand and (Path(cand).is_file() or shutil.which(cand)):
            return cand
    raise KernelError("no C++ compiler found (looked at $FLINT_CXX, $CXX, g++, c++, clang++); "
                      "the host runtime cannot be built and there is no fallback")


def _source_hash(name: str) -> str:
    h = hashlib.sha256()
    if name in HOST_MODULES:
        files, flags = [SRC_DIR / "host" / f"{name}.cpp"], HOST_FLAGS
    else:
        files, flags = sorted(SRC_DIR.glob("*.cuh")) + [SRC_DIR / f"{name}.cu"], NVCC_FLAGS
    for f in files:
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def _build_dirs():
    yield SRC_DIR / "_build"
    uid = os.getuid() if hasattr(os, "getuid") else 0
    yield Path(tempfile.gettempdir()) / f"flint_b200_build_{uid}"


def _writable(d: Path) -> bool:
    try:
        d.mkdir(parents=True, exist_ok=True)
        probe = d / f".probe_{os.getpid()}_{threading.get_ident()}"
        probe.write_bytes(b"")
        probe.unlink()
        return True
    except OSError:
        return False


def library_path(name: str) -> Path | None:
    """Path of an already built library for the current sources, if any."""
    tag = _source_hash(name)
    for d in _build_dirs():
        p = d / f"flint_{name}_{tag}.so"
        if p.is_file():
            return p
    return None


def compile_module(name: str, verbose: bool = True) -> Path:
    host = name in HOST_MODULES
    src = SRC_DIR / "host" / f"{name}.cpp" if host else SRC_DIR / f"{name}.cu"
    if not src.is_file():
        raise KernelError(f"no source {src}")
    found = library_path(name)
    if found is not None:
        return found
    out_dir = next((d for d in _build_dirs() if _writable(d)), None)
    if out_dir is None:
        raise KernelError("no writable folder for the compiled kernels (tried "
                          + ", ".join(str(d) for d in _build_dirs()) + ")")
    out = out_dir / f"flint_{name}_{_source_hash(name)}.so"
    tmp = out_dir / f".{out.name}.{os.getpid()}_{threading.get_ident()}.tmp"
    if host:
        cmd = [_host_compiler(), *HOST_FLAGS, "-o", str(tmp), str(src)]
    else:
        cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(SRC_DIR), "-o", str(tmp), str(src)]
    if verbose:
        print(f"[flint_b200] compiling {src.name}" + ("" if host else " for sm_100a") + " ...", file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def tick():
        while not done.wait(10.0):
            if verbose:
                print(f"[flint_b200]   {src.name}: still compiling ({time.time() - t0:.0f} s)",
                      file=sys.stderr, flush=True)
    th = threading.Thread(target=tick, daemon=True)
    th.start()
    log, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        try:
            tmp.unlink()
        except OSError:
            pass
        raise KernelError(f"the compiler failed on {src.name}:\n{log}")
    os.replace(tmp, out)
    if verbose:
        print(f"[flint_b200] compiled {src.name} in {time.time() - t0:.1f} s -> {out}", file=sys.stderr, flush=True)
    return out


def compile_all(names=None, verbose=True, jobs=4):
    """Compile several modules at once (used by the build check and by first use)."""
    names = list(names or available_modules())
    errors = {}
    paths = {}

    def work(n):
        try:
            paths[n] = compile_module(n, verbose)
        except Exception as e:  # collected and re-raised below
            errors[n] = e
    pending = list(names)
    while pending:
        batch, pending = pending[:jobs], pending[jobs:]
        ths = [threading.Thread(target=work, args=(n,)) for n in batch]
        for t in ths:
            t.start()
        for t in ths:
            t.join()
    if errors:
        raise KernelError("; ".join(f"{n}: {e}" for n, e in errors.items()))
    return paths


def load_module(name: str) -> ctypes.CDLL:
    with _LOCK:
        lib = _LOADED.get(name)
        if lib is None:
            path = compile_module(name)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise KernelError(f"cannot load {path}: {e}") from None
            _LOADED[name] = lib
        return lib
