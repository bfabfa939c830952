"""Plain, slow Phi-MoE forward pass: whole sequences, no cache, one function per part.

This file is the oracle of the test-suite.  It shares no code with ``flint_b200``:
it reads ``config.json`` as a dictionary and ``model.safetensors`` through its own
small reader, and computes everything with dense torch tensors on the CPU (float64
by default).  The reference project (formetaohy/Flint, crate family "Thuban") is
Rust + WGSL on wgpu and cannot be compiled or run here, and it has no MoE
feed-forward, so this file rests on formulas: the dense-decoder formulas are taken
from the reference files cited at each function, and the MoE feed-forward, the
LongRoPE mscale and the sliding window follow the architecture's definition
(top-2 sparsemixer over SiLU-gated w1/w3/w2 experts).
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

_ST_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
              "I32": torch.int32, "I64": torch.int64, "F64": torch.float64}


def read_safetensors(path):
    """Own reader: 8-byte little-endian header length, JSON header, raw tensor bytes."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = bytearray(raw[8 + n + lo:8 + n + hi])
        t = torch.frombuffer(buf, dtype=_ST_DTYPES[info["dtype"]]) if hi > lo else \
            torch.empty(0, dtype=_ST_DTYPES[info["dtype"]])
        out[name] = t.reshape(info["shape"]).clone()
    return out


def load_model_dir(model_dir, dtype=torch.float64):
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    tensors = {}
    for name, t in read_safetensors(model_dir / "model.safetensors").items():
        if name.startswith("model."):
            name = name[len("model."):]
        tensors[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, tensors


# ----------------------------------------------------------------------------- parts

def embed(ids, table):
    """h[r,:] = table[ids[r],:] * 1.0 (crates/thuban_kernel/wgsl/embed.wgsl:15-33,
    scale fixed to 1 for Phi: crates/thuban_architectures/src/transformer/config.rs:114)."""
    return table[torch.as_tensor(ids, dtype=torch.long)]


def layer_norm(x, gamma, beta, eps):
    """LayerNorm with bias, y=(x-mean)*rsqrt(var+eps)*gamma+beta
    (crates/thuban_kernel/wgsl/norm.wgsl:112-121, CPU twin
    crates/thuban_backend/tests/support/cpu_ref.rs:54-85).  The variance is taken as
    mean((x-mean)^2); it equals the reference's E[x^2]-mean^2 in exact arithmetic."""
    mu = x.mean(dim=-1, keepdim=True)
    var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
    y = (x - mu) / torch.sqrt(var + eps) * gamma
    return y + beta if beta is not None else y


def linear(x, w, b=None):
    """y[m,n] = sum_k x[m,k] * W[n,k] (+ b[n]) (crates/thuban_backend/tests/support/cpu_ref.rs:11-23,
    bias: crates/thuban_kernel/wgsl/bias.wgsl:11-16)."""
    y = x @ w.T
    return y + b if b is not None else y


def rope_scaling_of(cfg):
    rs = cfg.get("rope_scaling")
    if not rs:
        return None
    kind = rs.get("type", rs.get("rope_type", "longrope"))
    assert kind == "longrope", kind
    return rs


def rope_tables(cfg, head_dim, n_pos, dtype=torch.float64):
    """cos/sin tables [n_pos, rot/2]: inv_i = theta^(-2i/rot) / f_i with f the short
    factors for positions below the original context and the long factors from there
    on, chosen per position (crates/thuban_model/src/ops/rope.rs:52-87); the LongRoPE
    magnitude scale multiplies cos and sin."""
    rot = int(head_dim * cfg.get("partial_rotary_factor", 1.0))
    half = rot // 2
    theta = float(cfg["rope_theta"])
    i = torch.arange(half, dtype=torch.float64)
    inv = theta ** (-2.0 * i / rot)
    pos = torch.arange(n_pos, dtype=torch.float64)
    rs = rope_scaling_of(cfg)
    if rs is None:
        ang = pos[:, None] * inv[None, :]
        return torch.cos(ang).to(dtype), torch.sin(ang).to(dtype)
    orig = rs.get("original_max_position_embeddings",
                  cfg.get("original_max_position_embeddings", 4096))
    max_pos = cfg["max_position_embeddings"]
    default_m = math.sqrt(1.0 + math.log(max_pos / orig) / math.log(orig)) if max_pos > orig else 1.0
    m_short = rs.get("short_mscale", default_m)
    m_long = rs.get("long_mscale", default_m)
    short = torch.tensor(rs["short_factor"], dtype=torch.float64)
    long = torch.tensor(rs["long_factor"], dtype=torch.float64)
    is_short = (pos < orig)[:, None]
    inv_p = torch.where(is_short, inv / short, inv / long)
    msc = torch.where(is_short, torch.tensor(float(m_short), dtype=torch.float64),
                      torch.tensor(float(m_long), dtype=torch.float64))
    ang = pos[:, None] * inv_p
    return (torch.cos(ang) * msc).to(dtype), (torch.sin(ang) * msc).to(dtype)


def rope_rotate(x, cos, sin):
    """NeoX half-split rotation of x [T, heads, hd] by rows of cos/sin [T, rot/2]; dims
    at and above rot pass through (crates/thuban_kernel/wgsl/rope.wgsl:25-39,
    crates/thuban_backend/tests/support/cpu_ref.rs:132-151)."""
    half = cos.shape[-1]
    c, s = cos[:, None, :], sin[:, None, :]
    a, b, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
    return torch.cat([a * c - b * s, b * c + a * s, rest], dim=-1)


def attention(q, k, v, window):
    """Causal (and windowed) GQA attention over a whole sequence.  q [T,nq,hd],
    k,v [T,nkv,hd]; query at position p sees keys j with j<=p and, if window>0,
    j>=p+1-window; scale 1/sqrt(hd); softmax in full precision
    (crates/thuban_kernel/wgsl/attn.wgsl:78-90,119-214,
    crates/thuban_backend/tests/support/cpu_ref.rs:182-227)."""
    T, nq, hd = q.shape
    nkv = k.shape[1]
    g = nq // nkv
    scale = 1.0 / math.sqrt(hd)
    out = torch.zeros_like(q)
    p = torch.arange(T)
    allowed = p[None, :] <= p[:, None]
    if window and window > 0:
        allowed &= p[None, :] >= (p[:, None] + 1 - window)
    for h in range(nq):
        kh = h // g
        s = (q[:, h, :] @ k[:, kh, :].T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        out[:, h, :] = torch.softmax(s, dim=-1) @ v[:, kh, :]
    return out


def routing_fragility(scores, jitter_eps):
    """How close a row of router logits is to a point where the routing changes discontinuously:
    the smallest change of a single logit, as a fraction of the largest logit magnitude of the
    row, that would swap first and second or second and third place, or move a mask ratio
    (m - s_j) / max(|s_j|, m) across its threshold 2*eps.  A small value means that rounding
    elsewhere in the model may legitimately flip this decision."""
    s = scores
    sigma = s.abs().max().clamp(min=1e-30)
    top = torch.sort(s, descending=True).values
    d = [(top[0] - top[1]) / sigma]
    if s.numel() > 2:
        d.append((top[1] - top[2]) / sigma)
    i1 = int(torch.argmax(s))
    s2 = s.clone()
    s2[i1] = float("-inf")
    i2 = int(torch.argmax(s2))
    for m, skip in ((top[0], (i1,)), (top[1], (i1, i2))):
        factor = torch.clamp(s.abs(), min=m)
        ratio = (m - s) / factor
        need = (ratio - 2 * jitter_eps).abs() * factor / sigma      # change of s_j that reaches the threshold
        keep = torch.ones_like(s, dtype=torch.bool)
        for i in skip:
            keep[i] = False
        if keep.any():
            d.append(need[keep].min())
    return float(torch.stack(d).min())


def sparsemixer_top2(scores, jitter_eps):
    """Top-2 sparsemixer routing at inference, one row of router logits at a time.
    Returns (i1, g1, i2, g2); the two gates are not renormalised."""
    s = scores
    m1 = s.max()
    i1 = int(torch.argmax(s))          # lowest index on ties
    factor = torch.clamp(s.abs(), min=m1)
    mask1 = ((m1 - s) / factor) > (2.0 * jitter_eps)
    g1 = torch.softmax(s.masked_fill(mask1, float("-inf")), dim=-1)[i1]
    s2 = s.clone()
    s2[i1] = float("-inf")
    m2 = s2.max()
    i2 = int(torch.argmax(s2))
    factor2 = torch.clamp(s.abs(), min=m2)
    mask2 = ((m2 - s) / factor2) > (2.0 * jitter_eps)
    g2 = torch.softmax(s2.masked_fill(mask2, float("-inf")), dim=-1)[i2]
    return i1, g1, i2, g2


def activation(g, name):
    """silu(g)=g/(1+exp(-g)) or tanh-GELU (crates/thuban_kernel/wgsl/swiglu.wgsl:15-22,
    crates/thuban_backend/tests/support/cpu_ref.rs:102-108)."""
    if name == "silu":
        return g / (1.0 + torch.exp(-g))
    if name == "gelu_pytorch_tanh":
        return 0.5 * g * (1.0 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))
    raise ValueError(name)


def expert_mlp(x, w1, w3, w2, act="silu"):
    """y = (act(x W1^T) * (x W3^T)) W2^T (dense analogue:
    crates/thuban_model/src/ops/mlp.rs:24-79)."""
    return (activation(x @ w1.T, act) * (x @ w3.T)) @ w2.T


def moe_feed_forward(x, router_w, experts, jitter_eps, act="silu", record=None, forced=None):
    """x [T,H] -> sum over the two selected experts of gate * expert(x).

    The routing is decided token by token; each expert then runs once on all the rows that chose it
    (the same arithmetic per row as one call per token, and fast enough for real layer sizes).

    ``forced`` (tests of reduced-precision engines): per token an engine's decision
    (i1, i2, g1, g2).  Where it differs from this function's own decision, the engine's
    is used and the record notes the difference with this row's fragility, so that a test
    can require every difference to be a near-tie.  A record entry is (i1, i2, g1, g2, fragility,
    differs, this row's router logits)."""
    T = x.shape[0]
    logits = x @ router_w.T
    chosen = torch.zeros((T, 2), dtype=torch.long)
    gates = torch.zeros((T, 2), dtype=x.dtype)
    for t in range(T):
        i1, g1, i2, g2 = sparsemixer_top2(logits[t], jitter_eps)
        differs = False
        if forced is not None:
            f1, f2, fg1, fg2 = forced[t]
            differs = (f1, f2) != (i1, i2) or abs(fg1 - float(g1)) > 2e-2 or abs(fg2 - float(g2)) > 2e-2
            if differs:
                i1, i2, g1, g2 = f1, f2, fg1, fg2
        if record is not None:
            record.append((i1, i2, float(g1), float(g2), routing_fragility(logits[t], jitter_eps), differs, logits[t]))
        chosen[t, 0], chosen[t, 1] = i1, i2
        gates[t, 0], gates[t, 1] = g1, g2
    y = torch.zeros((2,) + tuple(x.shape), dtype=x.dtype)          # y[c, t] = expert chosen[t, c] applied to x[t]
    for e, (w1, w3, w2) in enumerate(experts):
        for c in range(2):
            rows = torch.nonzero(chosen[:, c] == e).flatten()
            if rows.numel():
                y[c, rows] = expert_mlp(x[rows], w1, w3, w2, act=act)
    return gates[:, 0:1] * y[0] + gates[:, 1:2] * y[1]


# ----------------------------------------------------------------------------- model

def norm_eps_of(cfg):
    for key in ("rms_norm_eps", "layer_norm_eps", "layer_norm_epsilon"):
        if key in cfg:
            return float(cfg[key])
    return 1e-5


def forward(cfg, w, token_ids, record_experts=None, forced_routing=None, logit_rows=None):
    """Logits [T, V] of one whole sequence (order of operations as
    crates/thuban_architectures/src/transformer/forward.rs:88-468).  ``logit_rows``: only these
    positions go through the final norm and the output head ([len(logit_rows), V])."""
    H = cfg["hidden_size"]
    nq = cfg["num_attention_heads"]
    nkv = cfg["num_key_value_heads"]
    hd = cfg.get("head_dim") or H // nq
    eps = norm_eps_of(cfg)
    E = cfg["num_local_experts"]
    jitter = cfg.get("router_jitter_noise", cfg.get("jitter_eps", 0.01))
    window = cfg.get("sliding_window") or 0
    act = cfg.get("hidden_act", "silu")
    T = len(token_ids)
    dtype = w["embed_tokens.weight"].dtype
    cos, sin = rope_tables(cfg, hd, T, dtype)

    h = embed(token_ids, w["embed_tokens.weight"])
    for l in range(cfg["num_hidden_layers"]):
        p = f"layers.{l}."
        x = layer_norm(h, w[p + "input_layernorm.weight"], w.get(p + "input_layernorm.bias"), eps)
        q = linear(x, w[p + "self_attn.q_proj.weight"], w.get(p + "self_attn.q_proj.bias"))
        k = linear(x, w[p + "self_attn.k_proj.weight"], w.get(p + "self_attn.k_proj.bias"))
        v = linear(x, w[p + "self_attn.v_proj.weight"], w.get(p + "self_attn.v_proj.bias"))
        q = rope_rotate(q.view(T, nq, hd), cos, sin)
        k = rope_rotate(k.view(T, nkv, hd), cos, sin)
        a = attention(q, k, v.view(T, nkv, hd), window).reshape(T, nq * hd)
        h = h + linear(a, w[p + "self_attn.o_proj.weight"], w.get(p + "self_attn.o_proj.bias"))
        x = layer_norm(h, w[p + "post_attention_layernorm.weight"],
                       w.get(p + "post_attention_layernorm.bias"), eps)
        experts = [(w[f"{p}block_sparse_moe.experts.{e}.w1.weight"],
                    w[f"{p}block_sparse_moe.experts.{e}.w3.weight"],
                    w[f"{p}block_sparse_moe.experts.{e}.w2.weight"]) for e in range(E)]
        rec = [] if record_experts is not None else None
        h = h + moe_feed_forward(x, w[p + "block_sparse_moe.gate.weight"], experts, jitter, act, rec,
                                 forced_routing[l] if forced_routing is not None else None)
        if record_experts is not None:
            record_experts.append(rec)
    if logit_rows is not None:
        h = h[torch.as_tensor(list(logit_rows), dtype=torch.long)]
    x = layer_norm(h, w["norm.weight"], w.get("norm.bias"), eps)
    head = w["embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return linear(x, head, w.get("lm_head.bias"))


def logits_for(model_dir, token_ids, dtype=torch.float64, round_to=None):
    """Convenience: load a model folder and run the whole sequence.  ``round_to``
    (e.g. torch.bfloat16) rounds the stored matrices first, to mimic a bf16 checkpoint."""
    cfg, w = load_model_dir(model_dir, dtype)
    if round_to is not None:
        w = {k: (t.to(round_to).to(dtype) if t.is_floating_point() else t) for k, t in w.items()}
    return forward(cfg, w, token_ids)


# ----------------------------------------------------------------------------- sampling

class PlainSampler:
    """Host sampler with the reference's order of operations
    (crates/thuban_generate/src/sampler.rs:56-109): repeat penalty, greedy if
    temperature<=0, softmax((s-max)/T), sort descending, top-k, top-p, min-p,
    renormalise, inverse-CDF draw with a splitmix64 step (:135-142)."""

    def __init__(self, temperature=0.7, top_k=20, top_p=0.8, min_p=0.0,
                 repeat_penalty=1.0, repeat_last_n=64, seed=42):
        self.t, self.k, self.p, self.min_p = temperature, top_k, top_p, min_p
        self.pen, self.last_n = repeat_penalty, repeat_last_n
        self.rng = seed & (2 ** 64 - 1)

    def next_f32(self):
        M = 2 ** 64 - 1
        self.rng = (self.rng + 0x9E3779B97F4A7C15) & M
        z = self.rng
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
        z ^= z >> 31
        return np.float32(z >> 40) / np.float32(1 << 24)

    def probs(self, logits, context=()):
        s = np.array(logits, dtype=np.float32).copy()
        if self.pen != 1.0 and len(context):
            for tok in list(context)[-self.last_n:] if self.last_n else []:
                if 0 <= tok < len(s):
                    s[tok] = s[tok] / np.float32(self.pen) if s[tok] > 0 else s[tok] * np.float32(self.pen)
        if self.t <= 0:
            return int(np.argmax(s)), None
        e = np.exp((s - s.max()) * np.float32(1.0 / self.t)).astype(np.float32)
        pr = e / e.sum(dtype=np.float32)
        order = np.argsort(-pr, kind="stable")
        kept = [(pr[i], int(i)) for i in order]
        if 0 < self.k < len(kept):
            kept = kept[:self.k]
        if self.p < 1.0:
            tot = np.float32(sum(v for v, _ in kept))
            acc, cut = np.float32(0), len(kept)
            for i, (v, _) in enumerate(kept):
                acc += v / tot
                if acc >= self.p:
                    cut = i + 1
                    break
            kept = kept[:max(cut, 1)]
        if self.min_p > 0 and kept:
            thr = np.float32(self.min_p) * kept[0][0]
            cut = next((i for i, (v, _) in enumerate(kept) if v < thr), len(kept))
            kept = kept[:max(cut, 1)]
        out = np.zeros_like(pr)
        for v, i in kept:
            out[i] = v
        return None, out / out.sum(dtype=np.float32)

    def sample(self, logits, context=()):
        tok, pr = self.probs(logits, context)
        if tok is not None:
            return tok
        u = self.next_f32()
        acc = np.float32(0)
        for i, v in enumerate(pr):
            acc += v
            if acc >= u:
                return i
        return len(pr) - 1
