"""Plain torch references for every kernel, with the kernels' own signatures.

Two uses: the ``-m gpu`` tests run each CUDA kernel beside its reference here, and the
CPU tests put this class in the place of the kernel set to exercise the engine's
plumbing (batching, cache, block tables, scheduler) without a GPU.  It is test code
only; the package never imports it.
"""
from __future__ import annotations

import math

import torch

from flint_b200.csrc.ops import MoePlan


def _act(g, name):
    if name == "silu":
        return g / (1.0 + torch.exp(-g))
    return 0.5 * g * (1.0 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))


class RefOps:
    name = "reference"

    def __init__(self, compute_dtype=torch.float32):
        self.cd = compute_dtype     # float64 gives an oracle for kernel tests
        self.launches = 0
        # the sampled tokens beside the two error flags, as the device kernels keep them
        self.MAX_TOKEN_ROWS = 256
        self.readback = torch.zeros(2 + self.MAX_TOKEN_ROWS, dtype=torch.int32)
        self.tc_error, self.page_error, self.token_out = self.readback[0:1], self.readback[1:2], self.readback[2:]

    # ------------------------------------------------------------------ row-wise
    def embed(self, ids, table, out, scale=1.0, fed_rows=None, fed_from=None):
        ids = ids.long()
        if fed_rows is not None:
            fed = fed_rows.long()
            ids = torch.where(fed >= 0, fed_from.to(fed.device).long()[fed.clamp(min=0)], ids)
        out.copy_((table[ids].to(self.cd) * scale).to(out.dtype))

    def norm(self, x, gamma, beta, eps, mode, out_f32=None, out_bf16=None, row_index=None):
        xs = x[row_index.long()] if row_index is not None else x
        xs = xs.to(self.cd)
        if mode == "layer":
            mu = xs.mean(-1, keepdim=True)
            var = ((xs - mu) ** 2).mean(-1, keepdim=True)
            y = (xs - mu) / torch.sqrt(var + eps) * gamma.to(self.cd)
            if beta is not None:
                y = y + beta.to(self.cd)
        else:
            y = xs / torch.sqrt((xs ** 2).mean(-1, keepdim=True) + eps) * gamma.to(self.cd)
        if out_f32 is not None:
            out_f32.copy_(y.to(torch.float32))
        if out_bf16 is not None:
            out_bf16.copy_(y.to(torch.float32).to(torch.bfloat16))

    def row_norm(self, x, gamma, beta, eps, mode, out_f32=None, out_bf16=None, row_index=None, pending=None,
                 router=None):
        if pending is not None:
            self.apply_pending(x, pending)
        if gamma is None:
            return
        tmp = out_f32
        if router is not None and tmp is None:
            tmp = torch.empty((x.shape[0], x.shape[1]), dtype=torch.float32)
        self.norm(x, gamma, beta, eps, mode, out_f32=tmp, out_bf16=out_bf16, row_index=row_index)
        if router is not None:
            self.router_sparsemixer(tmp, router.weight, router.jitter_eps, router.expert_ids, router.gates,
                                    getattr(router, "logits", None))

    def apply_pending(self, x, pending):
        if pending.partials is not None:
            add = pending.partials.to(self.cd).sum(0)
            if pending.bias is not None:
                add = add + pending.bias.to(self.cd)
            x.add_(add.to(x.dtype))
        if pending.y is not None:
            self.moe_combine(x, pending.y, pending.row_of, pending.gates)

    def gemm_partials(self, x, w, splits=None, plan=None):
        out = torch.empty((1, x.shape[0], w.shape[-2]), dtype=torch.float32)
        if plan is None:
            self.gemm(x, w, out[0])
        else:
            self.grouped_gemm(x, w, out[0], plan)
        return out

    def rope_kv_write(self, qkv, pos, slot, cos, sin, rot, q_out, cache, nq, nkv, hd, write_kv, status, bias=None,
                      style="half"):
        if qkv.dim() == 3:
            qkv = qkv.to(self.cd).sum(0)
        if bias is not None:
            qkv = qkv.to(self.cd) + bias.to(self.cd)
        T = qkv.shape[0]
        x = qkv.to(self.cd).view(T, nq + 2 * nkv, hd)
        half = rot // 2
        p = pos.long()

        def rotate(h):
            if rot == 0:
                return h
            c = cos[p].to(self.cd)[:, None, :]
            s = sin[p].to(self.cd)[:, None, :]
            if style == "interleaved":          # dims 2i and 2i + 1 rotate together
                a, b, rest = h[..., 0:rot:2], h[..., 1:rot:2], h[..., rot:]
                both = torch.stack([a * c - b * s, b * c + a * s], -1).reshape(*h.shape[:-1], rot)
                return torch.cat([both, rest], -1)
            a, b, rest = h[..., :half], h[..., half:rot], h[..., rot:]
            return torch.cat([a * c - b * s, b * c + a * s, rest], -1)
        q_out.copy_(rotate(x[:, :nq]).reshape(T, nq * hd).to(q_out.dtype))
        if not write_kv:
            return
        k = rotate(x[:, nq:nq + nkv])
        v = x[:, nq + nkv:]
        P = cache.page_size
        pages = cache.block_table[slot.long(), (p // P)].long()
        assert (pages >= 0).all(), "write to a position without a page"
        cache.k[pages, :, p % P, :] = k.to(cache.k.dtype)
        cache.v[pages, :, p % P, :] = v.to(cache.v.dtype)

    def gather_rows(self, x, index, out):
        idx = index.long()
        rows = x[idx.clamp(min=0)].clone()
        rows[idx < 0] = 0
        out.copy_(rows)

    def moe_combine(self, h, y, row_of, gates):
        r = row_of.view(-1, 2).long()
        g = gates.view(-1, 2).to(self.cd)
        yy = y.to(self.cd)
        h.add_((g[:, 0:1] * yy[r[:, 0]] + g[:, 1:2] * yy[r[:, 1]]).to(h.dtype))

    # ------------------------------------------------------------------ matrix products
    def gemm(self, x, w, out, bias=None, accumulate=False):
        y = x.to(self.cd) @ w.to(self.cd).T
        if bias is not None:
            y = y + bias.to(self.cd)
        if accumulate:
            y = y + out.to(self.cd)
        out.copy_(y.to(out.dtype))

    def _rows_by_expert(self, plan):
        off = plan.offsets.tolist()
        return [(e, off[e], off[e + 1]) for e in range(plan.n_experts) if off[e + 1] > off[e]]

    @staticmethod
    def pair_gate_up(w_gate, w_up):
        """This implementation keeps the gate rows before the up rows."""
        return torch.cat([w_gate, w_up], -2)

    def gated_gemm(self, x, w13, out, act="silu", plan=None):
        """w13 = pair_gate_up(gate, up): [2N, K] or [E, 2N, K]."""
        xs = x.to(self.cd)
        n = w13.shape[-2] // 2
        if plan is None:
            out.copy_((_act(xs @ w13[:n].to(self.cd).T, act) * (xs @ w13[n:].to(self.cd).T)).to(out.dtype))
            return
        for e, lo, hi in self._rows_by_expert(plan):
            g = xs[lo:hi] @ w13[e, :n].to(self.cd).T
            u = xs[lo:hi] @ w13[e, n:].to(self.cd).T
            out[lo:hi] = (_act(g, act) * u).to(out.dtype)

    def grouped_gemm(self, x, w, out, plan, plan_ready=False):
        xs = x.to(self.cd)
        for e, lo, hi in self._rows_by_expert(plan):
            out[lo:hi] = (xs[lo:hi] @ w[e].to(self.cd).T).to(out.dtype)

    # ------------------------------------------------------------------ attention
    def attention(self, q, cache, step, out, nq, nkv, hd, window, scale, tiling=None):
        self.paged_attention(q, cache, step.pos, step.slot, out, nq, nkv, hd, window, scale, step.max_kv_len)

    def paged_attention(self, q, cache, pos, slot, out, nq, nkv, hd, window, scale, max_kv_len, splits=None,
                        kernel=None, rows=None):
        T = q.shape[0]
        P = cache.page_size
        G = nq // nkv
        qq = q.to(self.cd).view(T, nq, hd)
        res = out.to(self.cd).view(T, nq, hd).clone()
        for t in (range(T) if rows is None else rows.tolist()):
            p = int(pos[t])
            lo = max(0, p + 1 - window) if window else 0
            js = torch.arange(lo, p + 1)
            pages = cache.block_table[int(slot[t]), js // P].long()
            assert (pages >= 0).all(), f"row {t}: key without a page"
            k = cache.k[pages, :, js % P, :].to(self.cd)      # [n, nkv, hd]
            v = cache.v[pages, :, js % P, :].to(self.cd)
            for h in range(nq):
                s = (k[:, h // G, :] @ qq[t, h]) * scale
                res[t, h] = torch.softmax(s, 0) @ v[:, h // G, :]
        out.copy_(res.reshape(T, nq * hd).to(out.dtype))

    def moe_tile_rows(self, n_tokens, n_experts, weight_dtype):
        return 64

    # ------------------------------------------------------------------ routing
    def router_sparsemixer(self, x, wr, eps, expert_ids, gates, logits_out=None):
        s_all = x.to(self.cd) @ wr.to(self.cd).T
        if logits_out is not None:
            logits_out.copy_(s_all.to(logits_out.dtype))
        for t in range(x.shape[0]):
            s = s_all[t]
            excluded = -1
            for r in range(2):
                cand = s.clone()
                if excluded >= 0:
                    cand[excluded] = float("-inf")
                m = cand.max()
                im = int(torch.argmax(cand))
                factor = torch.clamp(s.abs(), min=m)
                masked = ((m - s) / factor) > 2.0 * eps
                masked_scores = cand.masked_fill(masked, float("-inf"))
                expert_ids.view(-1, 2)[t, r] = im
                gates.view(-1, 2)[t, r] = torch.softmax(masked_scores, 0)[im].to(gates.dtype)
                excluded = im

    def moe_plan(self, expert_ids, n_experts, tile_rows):
        ids = expert_ids.reshape(-1).long()
        n = ids.numel()
        counts = torch.bincount(ids, minlength=n_experts)
        offsets = torch.zeros(n_experts + 1, dtype=torch.long)
        offsets[1:] = torch.cumsum(counts, 0)
        order = torch.argsort(ids, stable=True)
        row_of = torch.empty(n, dtype=torch.long)
        row_of[order] = torch.arange(n)
        token_of = order // 2
        tiles_e, tiles_r = [], []
        for e in range(n_experts):
            for r in range(0, int(counts[e]), tile_rows):
                tiles_e.append(e)
                tiles_r.append(int(offsets[e]) + r)
        max_tiles = n // tile_rows + min(n_experts, n)
        i32 = lambda t: torch.as_tensor(t, dtype=torch.int32)
        pad = lambda l: i32(l + [0] * (max_tiles - len(l)))
        return MoePlan(n_experts, tile_rows, max_tiles, i32(counts), i32(offsets), i32(row_of).view(-1, 2),
                       i32(token_of), pad(tiles_e), pad(tiles_r), i32([len(tiles_e)]))

    def moe_dispatch(self, expert_ids, n_experts, tile_rows, x):
        plan = self.moe_plan(expert_ids, n_experts, tile_rows)
        return plan, x[plan.token_of.long()].clone()

    # ------------------------------------------------------------------ sampling
    def argmax(self, logits, out):
        out.copy_(torch.argmax(logits, dim=-1).to(torch.int32))
