"""Python face of the CUDA kernels: one method per kernel, taking torch tensors.

``CudaOps`` checks types and shapes, hands raw pointers and the current stream to the
``extern "C"`` launchers and raises ``KernelError`` with the launcher's message on any
refusal.  It has no fallback: on a machine without the compiled extension or without
a CUDA device it raises.  The reference wraps its shaders the same way, one function
per shader building the scalar and binding lists (crates/thuban_model/src/ops/*.rs).
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from dataclasses import dataclass

import torch

from ..errors import KernelError
from . import build

F32, BF16 = 0, 1


def _raw_stream(device_index) -> int:
    """Handle of the device's current stream."""
    fast = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if fast is not None:
        return fast(device_index)
    return torch.cuda.current_stream(device_index).cuda_stream


def _code(dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


def _ptr(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def _check(t, name, dtype=None, dims=None, contiguous=True):
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name} must have {dims} dims, got shape {tuple(t.shape)}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


@dataclass
class MoePlan:
    """Rows sorted by expert: where each (token, choice) went and which expert owns each
    row tile.  All tensors live on the device; nothing is read back."""
    n_experts: int
    tile_rows: int
    max_tiles: int
    counts: torch.Tensor       # [E]
    offsets: torch.Tensor      # [E+1]
    row_of: torch.Tensor       # [T, 2] sorted row of (token, choice)
    token_of: torch.Tensor     # [2T] token of each sorted row
    tile_expert: torch.Tensor  # [max_tiles]
    tile_row0: torch.Tensor    # [max_tiles]
    n_tiles: torch.Tensor      # [1]


class CudaOps:
    """The kernel set on one CUDA device."""

    name = "cuda"

    def __init__(self, device="cuda:0"):
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: flint_b200 runs on the GPU only and has no CPU fallback")
        self.device = torch.device(device)
        self._device_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        # launch plans are sized for the device: so many blocks or warps per multiprocessor
        self.sm_count = int(torch.cuda.get_device_properties(self.device).multi_processor_count)
        self._libs = {}
        self.launches = 0
        self._profile = None
        self._label = None          # what the next launch works on (profiles list products by their shape)
        # One buffer for what the host reads back after a step, so that one copy brings all of it: a flag set by
        # a tensor-core kernel whose bounded wait ran out, a flag set by a kernel that met a position without a
        # page, and the sampled tokens.
        self.MAX_TOKEN_ROWS = 4096
        self.readback = torch.zeros(2 + self.MAX_TOKEN_ROWS, dtype=torch.int32, device=self.device)
        self.tc_error = self.readback[0:1]
        self.page_error = self.readback[1:2]
        self.token_out = self.readback[2:]
        # arrival counters of the decode attention kernels (one per row, kv head and chunk of query heads): zero
        # between launches; a launch that gave up a wait may leave some set, so they are cleared with its flag
        self.attention_arrivals = torch.zeros(1 << 15, dtype=torch.int32, device=self.device)

    # ------------------------------------------------------------------ plumbing
    def _fn(self, module, name):
        lib = self._libs.get(module)
        if lib is None:
            lib = build.load_module(module)
            getattr(lib, f"flint_{module}_last_error").restype = ctypes.c_char_p
            self._libs[module] = lib
        return getattr(lib, name)

    def _stream(self):
        """The current stream of the device as the launchers take it.  Asked for at every launch (a graph is
        captured on a stream of its own), through the call that returns the bare handle: building a stream
        object each time cost 7 us of the 25 us a launch takes on the host."""
        return c_void_p(_raw_stream(self._device_index))

    def _run(self, module, name, *args):
        fn = self._fn(module, name)
        if self._profile is not None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            rc = fn(*args, self._stream())
            e1.record()
            self._profile.append((name + (" " + self._label if self._label else ""), e0, e1))
        else:
            rc = fn(*args, self._stream())
        self._label = None
        self.launches += 1
        if rc != 0:
            msg = getattr(self._libs[module], f"flint_{module}_last_error")()
            raise KernelError((msg or b"unknown kernel error").decode())

    # Per-kernel device times, like the reference's timestamp profiler
    # (crates/thuban_profiler/src/lib.rs:173-248): events around every launch, summed by name.
    def start_profile(self):
        self._profile = []

    def stop_profile(self, ordered=False):
        """Returns {kernel name: (launches, total ms)} and stops profiling; ``ordered``: the launches in order
        instead, [(kernel name, ms)]."""
        torch.cuda.synchronize(self.device)
        if ordered:
            out = [(name, e0.elapsed_time(e1)) for name, e0, e1 in self._profile or []]
            self._profile = None
            return out
        out = {}
        for name, e0, e1 in self._profile or []:
            n, ms = out.get(name, (0, 0.0))
            out[name] = (n + 1, ms + e0.elapsed_time(e1))
        self._profile = None
        return out

    def wait_probe(self, limit_cycles=1_000_000):
        """Launch a kernel whose one wait, on a barrier nobody arrives at, runs out after ``limit_cycles`` clock
        cycles: it raises the same flag as a product kernel whose wait ran out, and returns.  Nothing faults or
        hangs.  For tests of the path from a kernel that gave up to the host's error."""
        self._run("gemm_tc", "flint_gemm_tc_wait_probe", c_longlong(int(limit_cycles)), _ptr(self.tc_error))

    def set_wait_cycles(self, cycles=0):
        """The limit (clock cycles) of every bounded wait in later launches of the tensor-core kernels;
        0 restores the default of about two seconds."""
        for module in ("gemm_tc", "attention_tc"):
            fn = self._fn(module, f"flint_{module}_set_wait_cycles")
            fn.restype = None
            fn(c_longlong(int(cycles)))

    def preload(self, modules=None):
        """Compile and load modules ahead of their first use."""
        mods = list(modules or build.available_modules())
        build.compile_all(mods)
        for m in mods:
            if m in build.MODULES:              # the host runtime is loaded by its own face
                self._fn(m, f"flint_{m}_last_error")

    # ------------------------------------------------------------------ row-wise
    def embed(self, ids, table, out, scale=1.0, fed_rows=None, fed_from=None):
        """Rows of the table by token id.  ``fed_rows`` [T] with ``fed_from``: where a row's entry is not
        negative, its token is read from that place of ``fed_from`` (tokens sampled on the device that the
        host has not read yet) instead of ``ids``."""
        _check(ids, "ids", torch.int32, 1)
        _check(table, "table", dims=2)
        _check(out, "out", torch.float32, 2)
        T, (V, H) = ids.numel(), table.shape
        if tuple(out.shape) != (T, H):
            raise KernelError(f"embed: out must be [{T}, {H}]")
        if (fed_rows is None) != (fed_from is None):
            raise KernelError("embed: fed rows and their source come together")
        if fed_rows is not None:
            _check(fed_rows, "fed_rows", torch.int32, 1)
            _check(fed_from, "fed_from", torch.int32, 1)
            if fed_rows.numel() != T:
                raise KernelError(f"embed: fed_rows must have {T} entries")
        self._run("elementwise", "flint_embed", _ptr(ids), _ptr(fed_rows), _ptr(fed_from), _ptr(table),
                  c_int(_code(table.dtype)), _ptr(out), c_int(T), c_int(H), c_int(V), c_float(scale))

    def norm(self, x, gamma, beta, eps, mode, out_f32=None, out_bf16=None, row_index=None):
        """mode 'layer' or 'rms'; writes float32 and/or bfloat16 copies of the result."""
        _check(x, "x", torch.float32, 2)
        H = x.shape[1]
        rows = row_index.numel() if row_index is not None else x.shape[0]
        _check(gamma, "gamma", torch.float32, 1)
        if gamma.numel() != H or (beta is not None and (beta.numel() != H or beta.dtype != torch.float32)):
            raise KernelError("norm: scale and bias must be float32 of the row width")
        for o, dt in ((out_f32, torch.float32), (out_bf16, torch.bfloat16)):
            if o is not None:
                _check(o, "norm output", dt, 2)
                if tuple(o.shape) != (rows, H):
                    raise KernelError(f"norm: output must be [{rows}, {H}]")
        if row_index is not None:
            _check(row_index, "row_index", torch.int32, 1)
        self._run("elementwise", "flint_norm", _ptr(x), _ptr(row_index), _ptr(gamma), _ptr(beta), c_float(eps),
                  c_int({"layer": 0, "rms": 1}[mode]), _ptr(out_f32), _ptr(out_bf16), c_int(rows), c_int(H))

    def row_norm(self, x, gamma, beta, eps, mode, out_f32=None, out_bf16=None, row_index=None, pending=None,
                 router=None):
        """Norm of the residual rows with what is pending applied first (x is updated in place) and,
        on request, the routing of every row.  Falls back to separate kernels for widths that the
        fused kernel does not take."""
        _check(x, "x", torch.float32, 2)
        T, H = x.shape
        if H % 4 or H > 16384 or (router is not None and (row_index is not None or H * 4 > 160000)):
            if pending is not None:
                self.apply_pending(x, pending)
            tmp = out_f32
            if router is not None and tmp is None:
                tmp = torch.empty((T, H), dtype=torch.float32, device=x.device)
            self.norm(x, gamma, beta, eps, mode, out_f32=tmp, out_bf16=out_bf16, row_index=row_index)
            if router is not None:
                self.router_sparsemixer(tmp, router.weight, router.jitter_eps, router.expert_ids, router.gates,
                                        getattr(router, "logits", None))
            return
        rows = row_index.numel() if row_index is not None else T
        for o, dt in ((out_f32, torch.float32), (out_bf16, torch.bfloat16)):
            if o is not None:
                _check(o, "norm output", dt, 2)
                if tuple(o.shape) != (rows, H):
                    raise KernelError(f"row_norm: output must be [{rows}, {H}]")
        if gamma is not None and (gamma.dtype != torch.float32 or gamma.numel() != H):
            raise KernelError("row_norm: scale must be float32 of the row width")
        partials = bias = y = row_of = gts = None
        S, stride = 0, 0
        if pending is not None:
            if pending.partials is not None:
                partials = pending.partials
                _check(partials, "pending partials", torch.float32, 3)
                if tuple(partials.shape[1:]) != (T, H):
                    raise KernelError("row_norm: pending partial sums do not match the residual")
                S, stride, bias = partials.shape[0], partials.stride(0), pending.bias
            if pending.y is not None:
                y, row_of, gts = pending.y, pending.row_of, pending.gates
                _check(y, "pending expert rows", torch.float32, 2)
                if y.shape[1] != H or row_of.numel() != 2 * T or gts.numel() != 2 * T:
                    raise KernelError("row_norm: pending expert rows do not match the residual")
        wr = logits = None
        E, jit, ids, gates = 0, 0.0, None, None
        if router is not None:
            wr, E, jit, ids, gates = router.weight, router.weight.shape[0], router.jitter_eps, router.expert_ids, router.gates
            logits = getattr(router, "logits", None)
            if logits is not None:
                _check(logits, "router logits", torch.float32, 2)
                if tuple(logits.shape) != (T, E):
                    raise KernelError(f"row_norm: router logits must be [{T}, {E}]")
            _check(wr, "router weight", dims=2)
            if wr.shape[1] != H or ids.numel() != 2 * T or gates.numel() != 2 * T:
                raise KernelError("row_norm: router shapes do not match")
        self._run("row_fused", "flint_row_norm", _ptr(x), _ptr(row_index), c_int(rows), c_int(H), _ptr(partials),
                  c_int(S), c_longlong(stride), _ptr(bias), _ptr(y), _ptr(row_of), _ptr(gts), _ptr(gamma), _ptr(beta),
                  c_float(eps), c_int({"layer": 0, "rms": 1}[mode]), _ptr(out_f32), _ptr(out_bf16), _ptr(wr),
                  c_int(_code(wr.dtype) if wr is not None else 0), c_int(E), c_float(jit), _ptr(ids), _ptr(gates),
                  _ptr(logits))

    def apply_pending(self, x, pending):
        """x += what a part left pending (for a norm that cannot take it along)."""
        _check(x, "x", torch.float32, 2)
        T, H = x.shape
        if H % 4 == 0 and H <= 16384:
            return self.row_norm(x, None, None, 0.0, "layer", pending=pending)
        if pending.partials is not None:
            p = pending.partials
            self._run("elementwise", "flint_add_partials", _ptr(x), _ptr(p), c_int(p.shape[0]), c_longlong(p.stride(0)),
                      _ptr(pending.bias), c_int(T), c_int(H))
        if pending.y is not None:
            self.moe_combine(x, pending.y, pending.row_of, pending.gates)

    def rope_kv_write(self, qkv, pos, slot, cos, sin, rot, q_out, cache, nq, nkv, hd, write_kv, status, bias=None,
                      style="half"):
        """qkv [T, W] or [S, T, W] float32 (S partial sums that are added here, with the bias).  ``style``: which
        dims of a head rotate together: "half" (i and i + rot/2) or "interleaved" (2i and 2i + 1)."""
        if style not in ("half", "interleaved"):
            raise KernelError(f"rope_kv_write: unknown rotation style {style!r}")
        if qkv.dim() == 2:
            qkv = qkv.unsqueeze(0)
        _check(qkv, "qkv", torch.float32, 3)
        S, T = qkv.shape[0], qkv.shape[1]
        if qkv.shape[2] != (nq + 2 * nkv) * hd:
            raise KernelError("rope_kv_write: qkv width does not match the head counts")
        if bias is not None and (bias.dtype != torch.float32 or bias.numel() != qkv.shape[2]):
            raise KernelError("rope_kv_write: bias must be float32 of the qkv width")
        _check(q_out, "q_out", dims=2)
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if cos.shape[1] * 2 != rot and rot > 0:
            raise KernelError("rope_kv_write: table width must be rot/2")
        if cache is not None:
            k, v, bt, P = cache.k, cache.v, cache.block_table, cache.page_size
            cdt = _code(k.dtype)
            if tuple(k.shape[1:]) != (nkv, P, hd) or tuple(v.shape[1:]) != (nkv, P, hd):
                raise KernelError(f"rope_kv_write: cache pages are {tuple(k.shape[1:])} and {tuple(v.shape[1:])}, "
                                  f"expected {(nkv, P, hd)} for both")
            max_pages = bt.shape[1]
        else:
            if write_kv:
                raise KernelError("rope_kv_write: no cache to write to")
            k = v = bt = None
            cdt, P, max_pages = F32, 16, 0
        self._run("elementwise", "flint_rope_kv_write", _ptr(qkv), _ptr(pos), _ptr(slot), _ptr(cos), _ptr(sin),
                  c_int(rot), c_int(1 if style == "interleaved" else 0), _ptr(q_out), c_int(_code(q_out.dtype)), _ptr(k),
                  _ptr(v), c_int(cdt), _ptr(bt),
                  c_int(max_pages), c_int(P), c_int(T), c_int(nq), c_int(nkv), c_int(hd), c_int(1 if write_kv else 0),
                  _ptr(status), c_int(S), c_longlong(qkv.stride(0)), _ptr(bias))

    def gather_rows(self, x, index, out):
        _check(x, "x", dims=2)
        _check(index, "index", torch.int32, 1)
        _check(out, "out", x.dtype, 2)
        if out.shape[0] != index.numel() or out.shape[1] != x.shape[1]:
            raise KernelError("gather_rows: output shape does not match")
        self._run("elementwise", "flint_gather_rows", _ptr(x), _ptr(index), _ptr(out), c_int(index.numel()),
                  c_int(x.shape[1] * x.element_size()))

    def moe_combine(self, h, y, row_of, gates):
        _check(h, "h", torch.float32, 2)
        _check(y, "y", torch.float32, 2)
        T, H = h.shape
        if y.shape[1] != H or row_of.numel() != 2 * T or gates.numel() != 2 * T:
            raise KernelError("moe_combine: shapes do not match")
        self._run("elementwise", "flint_moe_combine", _ptr(h), _ptr(y), _ptr(row_of), _ptr(gates), c_int(T), c_int(H))

    # ------------------------------------------------------------------ matrix products
    def gemm(self, x, w, out, bias=None, accumulate=False):
        """out = x @ w.T (+ bias) (+ out).  x [M,K], w [N,K], out [M,N]."""
        self._gemm(x, w, False, out, bias, accumulate, "silu", None)

    GATE_BLOCK = 16     # rows per block of the paired gate/up layout (GATE_BLOCK in common.cuh)

    @classmethod
    def paired_rows(cls, features):
        return 2 * -(-features // cls.GATE_BLOCK) * cls.GATE_BLOCK

    @classmethod
    def pair_gate_up(cls, w_gate, w_up):
        """The layout ``gated_gemm`` takes its weights in: blocks of 16 gate rows alternate with the 16 up
        rows of the same features; the feature count is padded to a multiple of 16 with zero rows.
        [..., N, K] twice -> [..., paired_rows(N), K]."""
        if w_gate.shape != w_up.shape:
            raise KernelError("pair_gate_up: gate and up weights differ in shape")
        *lead, n, k = w_gate.shape
        b = cls.GATE_BLOCK
        blocks = -(-n // b)
        out = w_gate.new_zeros((*lead, blocks, 2, b, k))
        flat = out.view(*lead, blocks, 2, b, k)
        pad = blocks * b - n
        for half, w in enumerate((w_gate, w_up)):
            if pad:
                w = torch.cat([w, w.new_zeros((*lead, pad, k))], -2)
            flat[..., half, :, :] = w.reshape(*lead, blocks, b, k)
        return out.view(*lead, 2 * blocks * b, k)

    def gated_gemm(self, x, w13, out, act="silu", plan: MoePlan | None = None):
        """out = act(x @ Wg.T) * (x @ Wu.T); w13 = pair_gate_up(Wg, Wu): [paired_rows(N), K], or with a
        plan (rows grouped by expert) [E, paired_rows(N), K]."""
        self._gemm(x, w13, True, out, None, False, act, plan)

    def grouped_gemm(self, x, w, out, plan: MoePlan, plan_ready=False):
        """out[r] = x[r] @ w[expert of row r].T; w [E, N, K].  ``plan_ready``: another product over the same plan
        has run since the plan was made (the kernel may then read the plan before it waits for the kernel before
        it, and fetch its first weights meanwhile)."""
        self._gemm(x, w, False, out, None, False, "silu", plan, plan_ready=plan_ready)

    def gemm_partials(self, x, w, splits=None, plan: MoePlan | None = None, plan_ready=False):
        """x @ w.T left as S partial sums over pieces of the K range: float32 [S, M, N], no bias.
        The next kernel (rotary write, row norm, gated activation) adds them up; S is 1 when nothing
        was split.  With a plan, rows are grouped by expert and w is [E, N, K]."""
        _check(x, "x", dims=2)
        _check(w, "w")
        M, K = x.shape
        N = w.shape[-2]
        if w.shape[-1] != K or (plan is None) != (w.dim() == 2):
            raise KernelError("gemm_partials: shapes do not match")
        if not self.tensor_core_ok(x, w, plan):
            out = torch.empty((1, M, N), dtype=torch.float32, device=x.device)
            self._gemm_simt(x, w, False, out[0], None, False, 0, plan, M, N, K)
            return out
        kb = -(-K // 64)
        stream_k = 0
        if plan is None:
            bn, E = self.token_tile(M), 1
            splits = splits or self._k_splits(M, N, K, bn)
        else:
            bn, E = plan.tile_rows, plan.n_experts
            if splits is None and bn <= 128 and kb >= 2:
                # few rows per expert: how many tiles there are is known on the device only, so the kernel
                # cuts the K blocks of all tiles into equal runs itself; a tile gets at most `splits` pieces
                stream_k, splits = 1, min(12, kb)
            splits = splits or 1
        if not stream_k:
            kbps = -(-kb // splits)
            splits = -(-kb // kbps)
        out = torch.empty((splits, M, N), dtype=torch.float32, device=x.device)
        self._label = self._product_label(N, K, plan, False)
        self._run("gemm_tc", "flint_gemm_tc", _ptr(x), c_int(x.stride(0)), _ptr(w), c_int(0), _ptr(None),
                  _ptr(out), c_int(F32), c_int(N), c_int(0), c_int(0), _ptr(plan.tile_expert if plan else None),
                  _ptr(plan.tile_row0 if plan else None), _ptr(plan.n_tiles if plan else None),
                  _ptr(plan.offsets if plan else None), c_int(plan.max_tiles if plan else 0), c_int(E), c_int(M),
                  c_int(N), c_int(K), c_int(bn), c_int(splits), _ptr(out), c_int(1), c_int(stream_k),
                  c_int(1 if plan_ready and plan is not None else 0), _ptr(self.tc_error))
        return out

    def _k_splits(self, M, N, K, bn):
        """Pieces of the K range so that a product with few tiles still fills the device."""
        tiles = -(-N // 128) * -(-M // bn)
        kb = -(-K // 64)
        if tiles >= self.sm_count or kb < 8:
            return 1
        # as many pieces as still fit one wave of resident blocks (three per SM with the 16-row token tile, whose
        # four stages take 72 KB, else two; a second, partial wave would cost as much as a full one: with the
        # 32-row tile counted at three, 17 to 32 rows ran 432 items on 296 places and a decode step took 1.5 % longer)
        return max(1, min(((3 if bn < 32 else 2) * self.sm_count) // tiles, kb // 4, 16))

    def _gemm(self, x, w, gated, out, bias, accumulate, act, plan, plan_ready=False):
        _check(x, "x", dims=2, contiguous=False)
        _check(out, "out", dims=2, contiguous=False)
        if x.stride(1) != 1 or out.stride(1) != 1:
            raise KernelError("gemm: rows must be contiguous")
        _check(w, "w")
        M, K = x.shape
        if plan is None:
            if w.dim() != 2:
                raise KernelError("gemm: dense weights must be [N, K]")
        elif w.dim() != 3 or w.shape[0] != plan.n_experts:
            raise KernelError("gemm: grouped weights must be [E, N, K]")
        N = out.shape[1] if gated else w.shape[-2]
        if gated and w.shape[-2] != self.paired_rows(N):
            raise KernelError(f"gemm: paired gate/up weights for {N} features have {self.paired_rows(N)} rows, "
                              f"not {w.shape[-2]}")
        if w.shape[-1] != K or tuple(out.shape) != (M, N):
            raise KernelError(f"gemm: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not match")
        if bias is not None:
            _check(bias, "bias", torch.float32, 1)
            if bias.numel() != N:
                raise KernelError("gemm: bias length does not match")
        act_code = {"silu": 0, "gelu_pytorch_tanh": 1}[act]
        if self.tensor_core_ok(x, w, plan):
            if gated and M <= 128:
                # few rows: the product is bound by streaming the weights, and a gated tile cannot split
                # its K range; run it as a plain product over the paired rows, split over K, and apply
                # the activation to the summed partial tiles
                parts = self.gemm_partials(x, w, plan=plan)
                self._run("elementwise", "flint_gated_act", _ptr(parts), c_int(parts.shape[0]),
                          c_longlong(parts.stride(0)), _ptr(out), c_int(_code(out.dtype)), c_int(M), c_int(N),
                          c_int(act_code))
                return
            self._gemm_tc(x, w, gated, out, bias, accumulate, act_code, plan, M, N, K, plan_ready)
        else:
            self._gemm_simt(x, w, gated, out, bias, accumulate, act_code, plan, M, N, K)

    # bfloat16 x bfloat16 with 16-byte aligned rows goes to the tensor cores; everything else
    # (float32 operands: the true 32-bit path; odd K) to the float32 pipes
    def tensor_core_ok(self, x, w, plan=None):
        return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
                and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
                and (plan is None or plan.tile_rows in (16, 32, 64, 128, 256)))

    @staticmethod
    def token_tile(rows):
        for bn in (16, 32, 64, 128):
            if rows <= bn:
                return bn
        return 256

    def moe_tile_rows(self, n_tokens, n_experts, weight_dtype):
        """Row-tile size the plan should use for grouped products over these weights."""
        if weight_dtype != torch.bfloat16:
            return 64
        return self.token_tile(-(-2 * n_tokens // n_experts))

    def _gemm_tc(self, x, w, gated, out, bias, accumulate, act_code, plan, M, N, K, plan_ready=False):
        if plan is not None:
            bn, splits, E = plan.tile_rows, 1, plan.n_experts
        else:
            E = 1
            bn = self.token_tile(M)
            splits = 1 if gated else self._k_splits(M, N, K, bn)
        partial = None
        if splits > 1:
            partial = torch.empty(splits * M * N, dtype=torch.float32, device=x.device)
        self._label = self._product_label(N, K, plan, gated)
        self._run("gemm_tc", "flint_gemm_tc", _ptr(x), c_int(x.stride(0)), _ptr(w), c_int(1 if gated else 0), _ptr(bias),
                  _ptr(out), c_int(_code(out.dtype)), c_int(out.stride(0)), c_int(1 if accumulate else 0),
                  c_int(act_code), _ptr(plan.tile_expert if plan else None), _ptr(plan.tile_row0 if plan else None),
                  _ptr(plan.n_tiles if plan else None), _ptr(plan.offsets if plan else None),
                  c_int(plan.max_tiles if plan else 0), c_int(E), c_int(M), c_int(N), c_int(K), c_int(bn),
                  c_int(splits), _ptr(partial), c_int(0), c_int(0), c_int(1 if plan_ready and plan is not None else 0),
                  _ptr(self.tc_error))

    @staticmethod
    def _product_label(N, K, plan, gated):
        """How a profile lists a product: its weight shape, and whether it is gated or over experts."""
        return f"{N}x{K}" + (" gated" if gated else "") + (" experts" if plan is not None else "")

    def _gemm_simt(self, x, w, gated, out, bias, accumulate, act_code, plan, M, N, K):
        if plan is not None and plan.tile_rows > 64:
            raise KernelError("gemm_simt: the plan's row tiles must not exceed 64 rows")
        self._label = self._product_label(N, K, plan, gated)
        self._run("gemm_simt", "flint_gemm_simt", _ptr(x), c_int(_code(x.dtype)), c_int(x.stride(0)), _ptr(w),
                  c_int(1 if gated else 0), c_int(_code(w.dtype)), _ptr(bias), _ptr(out), c_int(_code(out.dtype)),
                  c_int(out.stride(0)), c_int(1 if accumulate else 0), c_int(act_code),
                  _ptr(plan.tile_expert if plan else None), _ptr(plan.tile_row0 if plan else None),
                  _ptr(plan.n_tiles if plan else None), _ptr(plan.offsets if plan else None),
                  c_int(plan.max_tiles if plan else 0), c_int(plan.tile_rows if plan else 0), c_int(M), c_int(N), c_int(K))

    # ------------------------------------------------------------------ attention
    def attention_plan(self, T, nq, nkv, span, hd=128, bf16=True, ragged=True):
        """Which kernel and how to split the key range so that the device is filled:
        (kernel, keys per split, splits).  Few rows (decode), bfloat16, head sizes up to 128: the
        TMA-fed tensor-core kernel, one warp per (row, kv head, split); few rows otherwise: one block
        each on the float32 pipes; many rows: the warp-per-row kernel."""
        g_chunks = -(-(nq // nkv) // 4)
        base = T * nkv * g_chunks
        span = max(span, 1)
        if T <= 256 and hd <= 128 and bf16:
            # tensor-core decode kernel fed by TMA: 8 query heads per warp, at most one wave of 8 warps
            # per SM (a second, nearly empty wave would cost as much as a full one), at least 64 keys per warp
            base8 = T * nkv * -(-(nq // nkv) // 8)
            if span > 64 and (ragged or base8 >= 256 or (base8 >= 24 and base8 * span >= 24 * 16384)):
                # rows of different lengths, or many rows: the kernel cuts the keys of all rows into equal runs
                # itself; the count is the most pieces one (row, kv head) may be cut into: enough for one wave
                # of 8 warps per SM.  (Few rows of about the same length are a little faster with the key
                # range of each row cut into the same number of pieces, below; but from three rows on and about
                # 48 k keys in all, splits in fours leave part of the device idle, and equal runs win: measured
                # at 8 kv heads, of a decode step: 8 rows of 6,144 keys -4 %, of 8,192 -6 %, of 65,536 -19 %;
                # 16 rows of 3,072 -4 %, of 4,096 -5 %; 4 rows of 16,384 -3 %, of 65,536 -10 %; 3 rows of 32,768
                # -4 %; below that line the plan below is the faster by 1 to 3 %, and for two rows at any length.)
                return "stream", span, self._stream_slices(base8)
            n = max(1, min(span // 64, 8 * self.sm_count // base8))
            keys = -(-(-(-span // n)) // 16) * 16
            n = -(-span // keys)
            if n > 4 and n % 4:
                # splits in fours: the four warps of a block then hold one row's splits and merge them themselves
                # (the kernel divides a row's keys evenly over the splits; the last one may stay empty)
                n = n // 4 * 4
                keys = -(-(-(-span // n)) // 16) * 16
            if n == 4 and keys >= 384:
                # 19 to 31 rows of many keys: there is room for four to seven splits a row, and four leave up to
                # half of the warps without work while the others walk 24 steps and more; equal runs fill the
                # device (2,048 keys: -10 % of a decode step at 20 rows, -8 % at 24, -4 % at 28, -2 % at 31;
                # with 512 keys four splits of 8 steps are the faster)
                return "stream", span, self._stream_slices(base8)
            return "tma", keys, n
        if T <= 256:
            n = max(1, min(-(-span // 128), -(-8 * self.sm_count // base)))
            keys = -(-(-(-span // n)) // 128) * 128
            return "block", keys, -(-span // keys)
        if base >= 2048 or span <= 64:
            return "warp", span, 1
        n = min(-(-span // 64), -(-2048 // base))
        keys = -(-(-(-span // n)) // 32) * 32
        return "warp", keys, -(-span // keys)

    def _stream_slices(self, items):
        """The most pieces the stream kernel may cut one (row, kv head) item into: enough for one wave of
        8 warps per SM over all items."""
        return max(2, min(64, -(-8 * self.sm_count // items) + 1))

    def attention(self, q, cache, step, out, nq, nkv, hd, window, scale, tiling=None):
        """Attention of all rows of a step: long portions on the tensor cores (bfloat16, head
        sizes up to 128), decoded tokens and short portions row by row.  ``tiling``: the step's rows cut into
        tiles of up to 128 rows (``engine.step.Tiling``); without one every row goes row by row."""
        P = cache.page_size
        tc = (tiling is not None and tiling.n_tiles > 0 and q.dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16
              and hd <= 128 and (64 % P == 0 or P % 64 == 0) and step.attention_splits is None)
        if not tc:
            return self.paged_attention(q, cache, step.pos, step.slot, out, nq, nkv, hd, window, scale,
                                        step.max_kv_len, splits=step.attention_splits,
                                        ragged=not step.even_lengths, fresh_keys=step.longest_entry)
        self.attention_prefill_tc(q, cache, tiling.tiles, tiling.n_tiles, out, nq, nkv, hd, window, scale)
        if tiling.n_other_rows:
            self.paged_attention(q, cache, step.pos, step.slot, out, nq, nkv, hd, window, scale, step.max_kv_len,
                                 rows=tiling.other_rows, fresh_keys=step.longest_entry)

    def rope_attention_decode(self, qkv, bias, cos, sin, rot, style, cache, step, out, nq, nkv, hd, window, scale):
        """The rotary write and the attention of a batch of decoded tokens in one launch: qkv [S, T, W] float32
        (partial sums of the q/k/v projection, bias apart) becomes q, the rows' new keys and values go into the
        cache pages, and every row attends over its request's keys.  Returns False, having launched nothing, when
        the batch is not of the kind this kernel takes (then the caller runs the two kernels one after the
        other): it takes bfloat16 caches and outputs, head sizes up to 128, the half-split rotation, and batches
        whose requests are about equally long."""
        T = qkv.shape[1]
        if (style != "half" or step.attention_splits is not None or out.dtype != torch.bfloat16
                or cache.k.dtype != torch.bfloat16 or hd > 128 or step.n_tokens != len(step.entries) or T != step.n_tokens):
            return False
        span = min(step.max_kv_len, window) if window else step.max_kv_len
        kernel, keys, n = self.attention_plan(T, nq, nkv, span, hd, True, not step.even_lengths)
        g_chunks = -(-(nq // nkv) // 8)
        if kernel != "tma" or T * nkv * g_chunks > self.attention_arrivals.numel():
            return False
        if n % 4:
            # splits in fours: the four warps of a block share the row's queries and its new key and value
            n = max(4, n // 4 * 4)
            keys = -(-(-(-max(span, 1) // n)) // 16) * 16
        _check(qkv, "qkv", torch.float32, 3)
        _check(out, "out", torch.bfloat16, 2)
        if qkv.shape[2] != (nq + 2 * nkv) * hd or tuple(out.shape) != (T, nq * hd):
            raise KernelError("rope_attention_decode: widths do not match the head counts")
        if bias is not None and (bias.dtype != torch.float32 or bias.numel() != qkv.shape[2]):
            raise KernelError("rope_attention_decode: bias must be float32 of the qkv width")
        if tuple(cache.k.shape[1:]) != (nkv, cache.page_size, hd) or tuple(cache.v.shape[1:]) != (nkv, cache.page_size, hd):
            raise KernelError("rope_attention_decode: cache pages do not match the head counts")
        if rot and cos.shape[1] * 2 != rot:
            raise KernelError("rope_attention_decode: table width must be rot/2")
        scratch = torch.empty(T * nq * n * (hd + 2), dtype=torch.float32, device=qkv.device)
        self._run("attention_tc", "flint_attention_decode_fused", _ptr(qkv), c_int(qkv.shape[0]), c_longlong(qkv.stride(0)),
                  _ptr(bias), _ptr(cos), _ptr(sin), c_int(rot), _ptr(cache.k), _ptr(cache.v), c_int(cache.k.shape[0]),
                  _ptr(cache.block_table), c_int(cache.block_table.shape[1]), c_int(cache.page_size), _ptr(step.pos),
                  _ptr(step.slot), _ptr(out), c_int(T), c_int(nq), c_int(nkv), c_int(hd), c_int(window), c_float(scale),
                  c_int(keys), c_int(n), _ptr(scratch), _ptr(self.tc_error), _ptr(step.status),
                  _ptr(self.attention_arrivals), c_int(self.attention_arrivals.numel()))
        return True

    def attention_prefill_tc(self, q, cache, tiles, n_tiles, out, nq, nkv, hd, window, scale):
        _check(q, "q", torch.bfloat16, 2)
        _check(out, "out", torch.bfloat16, 2)
        _check(tiles, "tiles", torch.int32)
        T = q.shape[0]
        if q.shape[1] != nq * hd or tuple(out.shape) != (T, nq * hd):
            raise KernelError("attention_prefill_tc: q/out width does not match the head counts")
        if cache.k.dtype != torch.bfloat16 or tuple(cache.k.shape[1:]) != (nkv, cache.page_size, hd):
            raise KernelError("attention_prefill_tc: cache pages must be bfloat16 [page, kv head, P, head size]")
        self._run("attention_tc", "flint_attention_prefill_tc", _ptr(q), _ptr(cache.k), _ptr(cache.v),
                  c_int(cache.k.shape[0]), _ptr(cache.block_table), c_int(cache.block_table.shape[1]),
                  c_int(cache.page_size), _ptr(tiles), c_int(n_tiles), _ptr(out), c_int(T), c_int(nq), c_int(nkv),
                  c_int(hd), c_int(window), c_float(scale), _ptr(self.tc_error))

    def paged_attention(self, q, cache, pos, slot, out, nq, nkv, hd, window, scale, max_kv_len, splits=None,
                        kernel=None, rows=None, ragged=True, merge_in_kernel=True, fresh_keys=1 << 30):
        """rows: int32 list of the batch rows to compute (default: all).  ragged: the rows' key ranges may
        differ much in length (False: a decode batch whose requests are about equally long).
        merge_in_kernel (the tensor-core decode kernel with splits in fours): the pieces of a row's key range
        are merged by the block that finishes last; False: by a kernel of its own.
        fresh_keys: how many of a row's newest keys the kernel before this one in the stream may have written
        (1 for a batch of decoded tokens); the default assumes all of them."""
        _check(q, "q", dims=2)
        _check(out, "out", q.dtype, 2)
        T = q.shape[0]
        if q.shape[1] != nq * hd or tuple(out.shape) != (T, nq * hd):
            raise KernelError("paged_attention: q/out width does not match the head counts")
        if rows is not None:
            _check(rows, "rows", torch.int32, 1)
            T = rows.numel()
        if tuple(cache.k.shape[1:]) != (nkv, cache.page_size, hd):
            raise KernelError("paged_attention: cache pages do not match the head counts")
        span = min(max_kv_len, window) if window else max_kv_len
        auto_kernel, split_keys, n_splits = self.attention_plan(
            T, nq, nkv, span, hd, q.dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16, ragged)
        kernel = kernel or auto_kernel
        if splits is not None:
            split_keys, n_splits = splits
            if kernel == "stream":          # a given split is kept: the kernel with fixed key ranges
                kernel = "tma"
        if split_keys * n_splits < span:
            raise KernelError(f"paged_attention: {n_splits} splits of {split_keys} keys do not cover {span} keys")
        scratch = None
        if n_splits > 1:
            scratch = torch.empty(T * nq * n_splits * (hd + 2), dtype=torch.float32, device=q.device)
        arrivals = self.attention_arrivals if merge_in_kernel else None
        if kernel == "stream":
            if auto_kernel != "stream":
                n_splits = self._stream_slices(T * nkv * -(-(nq // nkv) // 8))
                scratch = torch.empty(T * nq * n_splits * (hd + 2), dtype=torch.float32, device=q.device)
            return self._run("attention_tc", "flint_attention_decode_stream", _ptr(q), _ptr(cache.k), _ptr(cache.v),
                             c_int(cache.k.shape[0]), _ptr(cache.block_table), c_int(cache.block_table.shape[1]),
                             c_int(cache.page_size), _ptr(pos), _ptr(slot), _ptr(out), c_int(T), c_int(nq), c_int(nkv),
                             c_int(hd), c_int(window), c_float(scale), c_int(n_splits), _ptr(scratch), _ptr(rows),
                             _ptr(self.tc_error), c_int(max(1, int(fresh_keys))))
        if kernel == "tma":
            if rows is not None and rows.numel() != T:
                raise KernelError("paged_attention: bad row list")
            return self._run("attention_tc", "flint_attention_decode_tc", _ptr(q), _ptr(cache.k), _ptr(cache.v),
                             c_int(cache.k.shape[0]), _ptr(cache.block_table), c_int(cache.block_table.shape[1]),
                             c_int(cache.page_size), _ptr(pos), _ptr(slot), _ptr(out), c_int(T), c_int(nq), c_int(nkv),
                             c_int(hd), c_int(window), c_float(scale), c_int(split_keys), c_int(n_splits),
                             _ptr(scratch), _ptr(rows), _ptr(self.tc_error), _ptr(arrivals),
                             c_int(arrivals.numel() if arrivals is not None else 0), c_int(max(1, int(fresh_keys))))
        fn = {"warp": "flint_paged_attention", "block": "flint_paged_attention_block"}[kernel]
        self._run("attention", fn, _ptr(q), c_int(_code(q.dtype)), _ptr(cache.k), _ptr(cache.v),
                  c_int(_code(cache.k.dtype)), _ptr(cache.block_table), c_int(cache.block_table.shape[1]),
                  c_int(cache.page_size), _ptr(pos), _ptr(slot), _ptr(out), c_int(_code(out.dtype)), c_int(T),
                  c_int(nq), c_int(nkv), c_int(hd), c_int(window), c_float(scale), c_int(split_keys), c_int(n_splits),
                  _ptr(scratch), _ptr(rows))

    # ------------------------------------------------------------------ routing
    def router_sparsemixer(self, x, wr, eps, expert_ids, gates, logits_out=None):
        _check(x, "x", torch.float32, 2)
        _check(wr, "router weight", dims=2)
        T, H = x.shape
        E = wr.shape[0]
        if wr.shape[1] != H:
            raise KernelError("router: weight width does not match")
        _check(expert_ids, "expert_ids", torch.int32)
        _check(gates, "gates", torch.float32)
        self._run("moe", "flint_router_sparsemixer", _ptr(x), _ptr(wr), c_int(_code(wr.dtype)), c_float(eps),
                  _ptr(expert_ids), _ptr(gates), _ptr(logits_out), c_int(T), c_int(H), c_int(E))

    def _plan_buffers(self, expert_ids, n_experts, tile_rows):
        _check(expert_ids, "expert_ids", torch.int32)
        n = expert_ids.numel()
        dev = expert_ids.device
        max_tiles = n // tile_rows + min(n_experts, n)
        ints = torch.empty(n_experts + (n_experts + 1) + n + n + 2 * max_tiles + 1, dtype=torch.int32, device=dev)
        o = 0
        parts = []
        for size in (n_experts, n_experts + 1, n, n, max_tiles, max_tiles, 1):
            parts.append(ints[o:o + size])
            o += size
        counts, offsets, row_of, token_of, tile_expert, tile_row0, n_tiles = parts
        plan = MoePlan(n_experts, tile_rows, max_tiles, counts, offsets, row_of.view(-1, 2), token_of,
                       tile_expert, tile_row0, n_tiles)
        return plan, [_ptr(t) for t in parts]

    def moe_plan(self, expert_ids, n_experts, tile_rows) -> MoePlan:
        plan, ptrs = self._plan_buffers(expert_ids, n_experts, tile_rows)
        self._run("moe", "flint_moe_plan", _ptr(expert_ids), c_int(expert_ids.numel()), c_int(n_experts),
                  c_int(tile_rows), *ptrs, c_int(plan.max_tiles))
        return plan

    def moe_dispatch(self, expert_ids, n_experts, tile_rows, x):
        """The plan for these choices and the rows of x in its order: (plan, xs) with
        xs[r] = x[plan.token_of[r]].  Few rows take one fused launch."""
        _check(x, "x", dims=2)
        n = expert_ids.numel()
        xs = torch.empty((n, x.shape[1]), dtype=x.dtype, device=x.device)
        row_bytes = x.shape[1] * x.element_size()
        if n > 256 or row_bytes % 16 or x.data_ptr() % 16:
            plan = self.moe_plan(expert_ids, n_experts, tile_rows)
            self.gather_rows(x, plan.token_of, xs)
            return plan, xs
        plan, ptrs = self._plan_buffers(expert_ids, n_experts, tile_rows)
        self._run("moe", "flint_moe_dispatch", _ptr(expert_ids), c_int(n), c_int(n_experts), c_int(tile_rows), *ptrs,
                  c_int(plan.max_tiles), _ptr(x), _ptr(xs), c_int(row_bytes))
        return plan, xs

    # ------------------------------------------------------------------ sampling
    def argmax(self, logits, out):
        _check(logits, "logits", torch.float32, 2)
        _check(out, "out", torch.int32, 1)
        self._run("sampling", "flint_argmax", _ptr(logits), _ptr(out), c_int(logits.shape[0]), c_int(logits.shape[1]))

    def sample(self, logits, params, context, work, out):
        """params [R, 8] float32: temperature, top_k, top_p, min_p, repeat_penalty, u, n_context, 0;
        context [R, C] int32 (recent tokens, -1 padded); work [R, V] float32 scratch."""
        _check(logits, "logits", torch.float32, 2)
        _check(params, "params", torch.float32, 2)
        _check(context, "context", torch.int32, 2)
        _check(work, "work", torch.float32, 2)
        _check(out, "out", torch.int32, 1)
        R, V = logits.shape
        if params.shape != (R, 8) or context.shape[0] != R or work.shape != (R, V) or out.numel() != R:
            raise KernelError("sample: shapes do not match")
        self._run("sampling", "flint_sample", _ptr(logits), _ptr(params), _ptr(context), c_int(context.shape[1]),
                  _ptr(work), _ptr(out), c_int(R), c_int(V))


_DEFAULT: dict = {}


def get_ops(device="cuda:0") -> CudaOps:
    key = str(torch.device(device))
    if key not in _DEFAULT:
        _DEFAULT[key] = CudaOps(device)
    return _DEFAULT[key]
