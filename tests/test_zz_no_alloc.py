"""The allocation-free attention entry point, called through its exported C symbol.

Some users of this library cannot allocate device memory when they call it (their process gave
all GPU memory to a pool of its own, or an allocation's device-wide synchronisation is not
acceptable where they stand).  ``flint_paged_attention_noalloc`` serves them: the partial results
of a split key range live in a 32 MiB array inside the library.  This test checks, on two calls
in a row that share that array, that it returns what the ordinary entry point returns and what a plain float64 attention over the same
cache gives, and that it refuses a shape whose scratch would not fit.  The file is named so that pytest collects it
last.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _args(q, k, v, bt, P, pos, slot, out, nq, nkv, hd, window, split_keys, n_splits):
    p = lambda t: c_void_p(t.data_ptr())
    code = 0 if q.dtype == torch.float32 else 1
    ccode = 0 if k.dtype == torch.float32 else 1
    return [p(q), c_int(code), p(k), p(v), c_int(ccode), p(bt), c_int(bt.shape[1]), c_int(P), p(pos), p(slot), p(out),
            c_int(code), c_int(q.shape[0]), c_int(nq), c_int(nkv), c_int(hd), c_int(window),
            c_float(1.0 / math.sqrt(hd)), c_int(split_keys), c_int(n_splits)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_noalloc_matches_the_ordinary_entry_point_twice_in_a_row(dtype):
    from flint_b200.cache.manager import CacheView, KVSpec
    from flint_b200.csrc import build
    from flint_b200.csrc.ops import get_ops
    from kernel_refs import RefOps
    ops = get_ops(DEV)
    lib = build.load_module("noalloc")
    lib.flint_noalloc_last_error.restype = ctypes.c_char_p
    lib.flint_paged_attention_noalloc_floats.restype = ctypes.c_longlong
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    nq, nkv, hd, P, n_pages = 8, 2, 64, 16, 40
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    g = torch.Generator().manual_seed(1)
    for call, (lens, window, split_keys) in enumerate([((300, 77, 150), 0, 64), ((41, 260, 9), 100, 32)]):
        k = torch.randn(n_pages, nkv, P, hd, generator=g).to(dtype).to(DEV)
        v = torch.randn(n_pages, nkv, P, hd, generator=g).to(dtype).to(DEV)
        bt = torch.full((3, 20), -1, dtype=torch.int32)
        perm = torch.randperm(n_pages, generator=g).to(torch.int32)
        o = 0
        for s, n in enumerate(lens):
            need = -(-n // P)
            bt[s, :need] = perm[o:o + need]
            o += need
        bt = bt.to(DEV)
        # a portion of 5 rows at the end of request 0 and one decoded token of each other request
        pos = torch.tensor(list(range(lens[0] - 5, lens[0])) + [lens[1] - 1, lens[2] - 1], dtype=torch.int32, device=DEV)
        slot = torch.tensor([0] * 5 + [1, 2], dtype=torch.int32, device=DEV)
        q = torch.randn(7, nq * hd, generator=g).to(dtype).to(DEV)
        span = min(max(lens), window) if window else max(lens)
        n_splits = -(-span // split_keys)
        assert n_splits > 1
        expected = torch.empty_like(q)
        ops.paged_attention(q, CacheView(k, v, bt, P, KVSpec(nkv, hd, window)), pos, slot, expected, nq, nkv, hd, window,
                            1.0 / math.sqrt(hd), max(lens), splits=(split_keys, n_splits))
        got = torch.full_like(q, float("nan"))
        rc = lib.flint_paged_attention_noalloc(*_args(q, k, v, bt, P, pos, slot, got, nq, nkv, hd, window, split_keys,
                                                      n_splits), stream)
        assert rc == 0, lib.flint_noalloc_last_error().decode()
        torch.cuda.synchronize()
        err = (got.double() - expected.double()).abs().max().item()
        assert err <= tol, f"call {call}: differs from the ordinary entry point by {err:.3e}"
        # and against arithmetic that shares nothing with either entry point
        plain = torch.zeros(q.shape, dtype=torch.float64)
        RefOps(torch.float64).paged_attention(q.cpu(), CacheView(k.cpu(), v.cpu(), bt.cpu(), P, KVSpec(nkv, hd, window)),
                                              pos.cpu(), slot.cpu(), plain, nq, nkv, hd, window, 1.0 / math.sqrt(hd),
                                              max(lens))
        err = (got.double().cpu() - plain).abs().max().item()
        assert err <= tol, f"call {call}: differs from the plain attention by {err:.3e}"
    # a shape beyond the built-in array is refused with a clear error, and nothing runs
    big_T, big_splits = 4096, 64
    assert lib.flint_paged_attention_noalloc_floats(big_T, nq, hd, big_splits) * 4 > 32 * 1024 * 1024
    a = _args(q, k, v, bt, P, pos, slot, got, nq, nkv, hd, 0, 8, big_splits)
    a[12] = c_int(big_T)
    rc = lib.flint_paged_attention_noalloc(*a, stream)
    assert rc != 0 and b"scratch" in lib.flint_noalloc_last_error()
