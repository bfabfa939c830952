#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Phi-mini-MoE layer sizes, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints one JSON line.  ``value`` is decoded tokens per second at batch 8 (a "step" is
one decode step of the whole batch, timed on the device with CUDA events); ``e2e`` is
the same through ``Engine.step`` with host tokens in and out; ``prefill`` is one
2,048-token prompt; ``roofline`` relates the bytes a decode step must read to its time;
``points`` has decode at batch 1 and 64.  The engine runs on one GPU: for ``--gpus N``
with N > 1 it says so and exits with 2.
"""
import argparse
import json
import os
import random
import statistics
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

# Phi-mini-MoE layer sizes (the third configuration of BASELINE.json)
MINI = {
    "architectures": ["PhimoeForCausalLM"], "model_type": "phimoe",
    "vocab_size": 32064, "hidden_size": 4096, "intermediate_size": 960, "num_hidden_layers": 32,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "max_position_embeddings": 131072, "original_max_position_embeddings": 4096, "rope_theta": 10000.0,
    "sliding_window": 131072, "rms_norm_eps": 1e-5, "hidden_act": "silu",
    "attention_bias": True, "lm_head_bias": True, "tie_word_embeddings": False,
    "num_local_experts": 16, "num_experts_per_tok": 2, "router_jitter_noise": 0.01,
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def peaks():
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            d = json.load(open(path))
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
        except (ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


def mini_config(layers=None, expert_intermediate=None, sizes=None):
    """The Phi-mini-MoE sizes, with any of them replaced (``sizes``: config.json key -> value)."""
    cfg = dict(MINI)
    if expert_intermediate:
        cfg["intermediate_size"] = int(expert_intermediate)
    for key, value in (sizes or {}).items():
        if value:
            cfg[key] = int(value)
    r = random.Random(7)
    half = cfg["head_dim"] // 2
    cfg["rope_scaling"] = {"type": "longrope",
                           "short_factor": [round(r.uniform(1, 4), 4) for _ in range(half)],
                           "long_factor": [round(r.uniform(1, 4), 4) for _ in range(half)]}
    if layers:
        cfg["num_hidden_layers"] = layers
    return cfg


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
        sm = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v == "Active"})
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def build_model(cfg, max_slots, ctx, device="cuda:0", n_pages=None):
    import torch
    from flint_b200.engine.loading import expected_from_config
    from flint_b200.engine.model import Model
    from flint_b200.weights.sources import RandomSource
    spec, expected = expected_from_config(cfg)
    src = RandomSource(expected, seed=0, dtype=torch.bfloat16, on_device=True)
    return Model(spec, src, dtype="bfloat16", device=device, page_size=64, n_pages=n_pages or max_slots * (ctx // 64),
                 max_slots=max_slots, max_context=ctx, max_step_tokens=2048 + max_slots)


def checked(model, logits, what):
    """A timed region counts only if no kernel raised a flag in it (a bounded wait that ran out, a position
    without a page) and its last logits are finite numbers."""
    import torch
    model.check_status()
    if logits is not None and not bool(torch.isfinite(logits).all()):
        raise SystemExit(f"bench.py: {what} produced logits that are not finite; no number is reported")


def step_flops(cfg, n_tokens, kv_lens):
    """Multiply-add flops x2 of one step: projections, attention over the cache, router, two experts."""
    H, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    nq, nkv, hd, E = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["num_local_experts"]
    per_tok = 2 * H * (nq + 2 * nkv) * hd + 2 * nq * hd * H + 2 * H * E + 2 * (3 * H * I) * 2
    attn = sum(4 * nq * hd * k for k in kv_lens)       # QK^T and PV per (token, keys seen)
    return L * (n_tokens * per_tok + attn)


def decode_bytes(cfg, model, batch_kv_lens, distinct_experts):
    """Bytes a decode step must read: every weight it uses once, and the live requests' cache."""
    H, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    nq, nkv, hd, E, V = (cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                         cfg["num_local_experts"], cfg["vocab_size"])
    attn_w = ((nq + 2 * nkv) * hd * H + nq * hd * H) * 2
    router = E * H * 2
    expert = 3 * H * I * 2
    weights = L * (attn_w + router) + sum(distinct_experts) * expert + V * H * 2
    kv = sum(batch_kv_lens) * nkv * hd * 2 * 2 * L
    return weights + kv


def run_decode(model, cfg, batch, prompt_len, steps, warmup, rng, count_experts=True):
    """Prefill ``batch`` requests of ``prompt_len`` random tokens, then time decode steps."""
    import torch
    from flint_b200.engine.step import StepEntry
    V = cfg["vocab_size"]
    slots = [model.cache.admit() for _ in range(batch)]
    for s in slots:
        model.cache.ensure(s, 0, prompt_len)
        for p0 in range(0, prompt_len, 2048):          # in portions, as the scheduler would
            n = min(2048, prompt_len - p0)
            model.step([StepEntry(s, p0, [rng.randrange(V) for _ in range(n)], [])])
    pos = prompt_len
    distinct = None
    if count_experts:
        rec = {}
        for s in slots:
            model.cache.ensure(s, pos, pos + 1)
        model.step([StepEntry(s, pos, [rng.randrange(V)], [0]) for s in slots], record=rec)
        distinct = [int(torch.unique(ids).numel()) for ids in rec["experts"]]
        pos += 1

    def one():
        nonlocal pos
        for s in slots:
            model.cache.ensure(s, pos, pos + 1)
        out = model.step([StepEntry(s, pos, [rng.randrange(V)], [0]) for s in slots])
        pos += 1
        return out
    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    l0 = model.ops.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        last = one()
    e1.record()
    torch.cuda.synchronize()
    checked(model, last, f"decoding at batch {batch}")
    ms = e0.elapsed_time(e1) / steps
    launches = model.ops.launches - l0
    kv_lens = [pos] * batch
    for s in slots:
        model.cache.release(s)
    return {"ms": ms, "tok_s": batch * 1000.0 / ms, "launches": launches, "distinct": distinct, "kv_lens": kv_lens}


def run_prefill(model, cfg, n_tokens, reps, warmup, rng):
    import torch
    from flint_b200.engine.step import StepEntry
    V = cfg["vocab_size"]
    times = []
    for i in range(warmup + reps):
        s = model.cache.admit()
        toks = [rng.randrange(V) for _ in range(n_tokens)]
        model.cache.ensure(s, 0, n_tokens)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        last = model.step([StepEntry(s, 0, toks, [n_tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        checked(model, last, f"the prefill of {n_tokens} tokens")
        if i >= warmup:
            times.append(e0.elapsed_time(e1))
        model.cache.release(s)
    return statistics.median(times)


def run_e2e(model, cfg, batch, prompt_len, steps, warmup, rng):
    """The same decode through the public entry point: Engine.step, host tokens in and out."""
    import torch
    from flint_b200.engine.engine import Engine
    from flint_b200.sampling.params import SamplingParams
    eng = Engine(model, SamplingParams.greedy(), seed=1, prefill_chunk=2048, max_step_tokens=2048 + batch)
    V = cfg["vocab_size"]
    # prompts go in one portion per step, so the first request has decoded batch * portions tokens before the
    # last one is in: give all of them room to keep decoding through the timed region
    portions = -(-prompt_len // 2048)
    ids = [eng.create([rng.randrange(V) for _ in range(prompt_len)], steps + warmup + batch * (portions + 1) + 8)
           for _ in range(batch)]
    while any(r.remaining > 1 for r in eng.scheduler.running) or eng.scheduler.waiting:
        eng.step()
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n_tok = 0
    for _ in range(steps):
        n_tok += eng.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    h2d = model.staging.host.numel() * 4
    for i in ids:
        eng.close(i)
    return {"tok_s": n_tok / dt, "h2d": h2d, "d2h": (batch + 2) * 4, "ms": dt * 1000 / steps}


def run_mixed(model, cfg, n_requests, lo, hi, decode_tokens, rng):
    """Continuous batching through the engine: requests with prompts of lo..hi random tokens, all submitted
    at once, each decoding ``decode_tokens`` tokens greedily; wall time from the first step to the last."""
    import torch
    from flint_b200.engine.engine import Engine
    from flint_b200.sampling.params import SamplingParams
    eng = Engine(model, SamplingParams.greedy(), seed=1, prefill_chunk=2048, max_step_tokens=2048 + n_requests)
    V = cfg["vocab_size"]
    lens = [rng.randint(lo, hi) for _ in range(n_requests)]
    ids = [eng.create([rng.randrange(V) for _ in range(n)], decode_tokens) for n in lens]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    steps = 0
    while eng.has_work():
        eng.step()
        steps += 1
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    stats = [eng.stats(i) for i in ids]
    for i in ids:
        eng.close(i)
    return {"seconds": dt, "steps": steps, "prompt_tokens": sum(lens), "decoded": sum(s.decode_tokens + 1 for s in stats),
            "preemptions": sum(s.preemptions for s in stats)}


def run_long(cfg, pk, rng, lengths, decode_tokens, chunk=2048):
    """Long contexts (the last configuration of BASELINE.json): prompts of ``lengths`` tokens run in portions of
    ``chunk`` through the step function, each portion timed with its depth; then ``decode_tokens`` steps of all
    requests together; then the same workload through ``Engine`` (continuous batching: a request decodes while
    the next one's prompt runs), wall clock."""
    import torch
    from flint_b200.engine.engine import Engine
    from flint_b200.engine.step import StepEntry
    from flint_b200.sampling.params import SamplingParams
    V = cfg["vocab_size"]
    ctx = max(lengths) + decode_tokens
    n_pages = sum(-(-(n + decode_tokens) // 64) for n in lengths) + 8
    model = build_model(cfg, len(lengths), ctx, n_pages=n_pages)
    by_depth = {}
    slots = []
    t_prefill = 0.0
    for n in lengths:
        s = model.cache.admit()
        slots.append(s)
        model.cache.ensure(s, 0, n)
        for p0 in range(0, n, chunk):
            m = min(chunk, n - p0)
            toks = [rng.randrange(V) for _ in range(m)]
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            last = model.step([StepEntry(s, p0, toks, [m - 1] if p0 + m == n else [])])
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            t_prefill += ms
            if m == chunk:
                by_depth.setdefault(p0, []).append(ms)
        checked(model, last, f"the prefill of {n} tokens")
    depth_points = {}
    for d in (0, 4096, 16384, 32768 - chunk, 65536, max(lengths) // chunk * chunk - chunk):
        if d in by_depth:
            depth_points[f"prefill_tok_s_at_depth_{d}"] = round(chunk * 1000.0 / statistics.median(by_depth[d]), 1)
    pos = list(lengths)

    def one(record=None):
        for i, s in enumerate(slots):
            model.cache.ensure(s, pos[i], pos[i] + 1)
        out = model.step([StepEntry(s, pos[i], [rng.randrange(V)], [0]) for i, s in enumerate(slots)], record=record)
        for i in range(len(pos)):
            pos[i] += 1
        return out
    rec = {}
    one(rec)
    distinct = [int(torch.unique(ids).numel()) for ids in rec["experts"]]
    for _ in range(3):
        one()
    torch.cuda.synchronize()
    n_timed = decode_tokens - 4
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n_timed):
        last = one()
    e1.record()
    torch.cuda.synchronize()
    checked(model, last, "decoding at long contexts")
    ms = e0.elapsed_time(e1) / n_timed
    bytes_step = decode_bytes(cfg, model, pos, distinct)
    for s in slots:
        model.cache.release(s)
    # as served: all requests submitted at once
    eng = Engine(model, SamplingParams.greedy(), seed=1, prefill_chunk=chunk, max_step_tokens=chunk + len(lengths))
    ids = [eng.create([rng.randrange(V) for _ in range(n)], decode_tokens) for n in lengths]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    while eng.has_work():
        eng.step()
    torch.cuda.synchronize()
    served = time.perf_counter() - t0
    stats = [eng.stats(i) for i in ids]
    errors = [eng.error(i) for i in ids if eng.error(i)]
    for i in ids:
        eng.close(i)
    if errors:
        raise SystemExit(f"bench.py: the served run failed: {errors[0]}")
    return {"metric": f"long contexts: prompts of {', '.join(f'{n:,}' for n in lengths)} tokens in portions of {chunk:,}, "
                      f"then {decode_tokens} decoded tokens each",
            "value": round(sum(lengths) * 1000.0 / t_prefill, 1), "unit": "prompt tokens/s (all portions, device time)",
            **depth_points,
            "decode_ms_per_step": round(ms, 3), "decode_tok_s": round(len(lengths) * 1000.0 / ms, 1),
            "decode_roofline_frac": round(bytes_step / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4),
            "decode_bytes_per_step": bytes_step, "cache_tokens": sum(pos),
            "served_seconds": round(served, 2), "served_tok_s": round((sum(lengths) + sum(s.decode_tokens + 1 for s in stats)) / served, 1),
            "config": config_of(cfg, len(lengths), max(lengths), ctx, pk)}


def run_sweep(cfg, pk, rng, steps, warmup):
    """``--sweep``: decode at further batch sizes and context lengths, each with its roofline fraction: batch 1 and
    8 at contexts of 16,384 and 65,536 tokens, batch 1 at 131,008, and batch 128 and 256 at 2,048.  One model, the
    cache sized for the largest point (about 70 GB)."""
    import torch
    points = [(1, 16384), (8, 16384), (1, 65536), (8, 65536), (1, 131072 - 64), (128, 2048), (256, 2048)]
    n_pages = max(b * -(-(c + 64) // 64) for b, c in points) + 8
    model = build_model(cfg, max(b for b, _ in points), 131072, n_pages=n_pages)
    out = {}
    for b, c in points:
        r = run_decode(model, cfg, b, c, steps, warmup, rng)
        frac = decode_bytes(cfg, model, r["kv_lens"], r["distinct"]) / (r["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"]
        out[f"decode_b{b}_ctx{c}"] = {"tok_s": round(r["tok_s"], 1), "ms_per_step": round(r["ms"], 3),
                                      "roofline_frac": round(frac, 4)}
        torch.cuda.empty_cache()
    return {"metric": "decode tok/s at further batch sizes and context lengths", "points": out,
            "config": config_of(cfg, 0, 0, 131072, pk)}


def run_tiny(which, reps=5):
    """The tiny workloads of the two test configurations, in 32-bit: through ``Engine`` on the GPU (wall clock,
    host tokens in and out) and on the timed CPU baseline, the plain C++ implementation of the test-suite
    (tests/plain_phimoe.cpp: float32, whole-sequence forward pass for every token, one thread)."""
    import tempfile
    import torch
    sys.path.insert(0, os.path.join(REPO, "tests"))
    import plain_cpp
    import tiny
    from flint_b200.engine.engine import Engine
    from flint_b200.engine.model import load_model
    from flint_b200.sampling.params import SamplingParams
    cfg = tiny.CONFIGS[which]
    if which == "A":
        lens, n_tokens, params, chunk = (7, 13, 32), 16, SamplingParams.greedy(), 2048
    else:
        lens, n_tokens, params, chunk = (5, 40, 70, 100), 24, SamplingParams(temperature=0.8, top_k=20, top_p=0.8), 16
    prompts = [tiny.random_tokens(n, cfg["vocab_size"], 100 + n) for n in lens]
    with tempfile.TemporaryDirectory() as d:
        folder = tiny.write_tiny(os.path.join(d, "tiny"), which, seed=0, dtype=torch.float32)
        base_tokens, base_secs = plain_cpp.generate(folder, prompts, n_tokens, params.temperature, params.top_k,
                                                    params.top_p, seed=42)
        model = load_model(folder, dtype="float32", page_size=16, n_pages=64, max_slots=len(prompts), max_step_tokens=256)
        times = []
        for i in range(reps + 2):
            eng = Engine(model, params, seed=42, prefill_chunk=chunk, stop=())
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            got = eng.generate(prompts, n_tokens)
            torch.cuda.synchronize()
            if i >= 2:
                times.append(time.perf_counter() - t0)
        model.check_status()
    n_out = sum(len(g) for g in got)
    ours = n_out / statistics.median(times)
    base = sum(len(g) for g in base_tokens) / base_secs
    return {"metric": f"generated tokens/s, Tiny {which} workload ({len(prompts)} requests, prompts of "
                      f"{'/'.join(map(str, lens))} tokens, {n_tokens} tokens each, "
                      f"{'greedy' if params.temperature <= 0 else 'temperature 0.8, seed 42'})",
            "value": round(ours, 1), "unit": "tokens/s", "n_gpus": 1, "dtype": "fp32", "higher_is_better": True,
            "vs_baseline": round(ours / base, 2),
            "baseline": {"impl": "tests/plain_phimoe.cpp: plain float32 C++, whole-sequence forward pass per token, one CPU thread",
                         "value": round(base, 1), "seconds": round(base_secs, 4)},
            "tokens_match_baseline": got == base_tokens, "seconds": round(statistics.median(times), 5),
            "data": "synthetic: seeded random weights, uniform-random token ids", "impl": "ours"}


def config_of(cfg, batch, prompt_tokens, ctx, pk):
    """Every size of a run, flat."""
    mini = all(cfg[k] == MINI[k] for k in MINI if k != "num_hidden_layers")
    return {"model": "Phi-mini-MoE sizes" if mini else
                     f"Phi-MoE sizes: hidden {cfg['hidden_size']}, experts of {cfg['intermediate_size']}",
            "layers": cfg["num_hidden_layers"], "layers_of_config": 32,
            "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"], "experts": cfg["num_local_experts"],
            "top_k": 2, "expert_intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "global_batch": batch, "prompt_tokens": prompt_tokens, "seq_len": ctx, "page_size": 64,
            "parallelism": "single GPU", "l2": "inputs larger than L2 (weights streamed every step)",
            "peaks": pk["source"]}


def profile_tables(model, cfg, batch, prompt_len, rng):
    """Per-kernel device time (CUDA events around every launch, graphs off, so launches are serialised): one
    prefill of ``prompt_len`` tokens and one decode step of the batch at that context.  Returns
    (prefill table, decode table, distinct experts per layer of the decode step), tables as
    {launcher name and product shape: (launches, ms)}."""
    import torch
    from flint_b200.engine.step import StepEntry
    V = cfg["vocab_size"]
    graphs, model.use_graphs = model.use_graphs, False
    slots = [model.cache.admit() for _ in range(batch)]
    for i, s in enumerate(slots):
        model.cache.ensure(s, 0, prompt_len + 2)
        if i == len(slots) - 1:
            model.ops.start_profile()
        model.step([StepEntry(s, 0, [rng.randrange(V) for _ in range(prompt_len)], [prompt_len - 1])])
    prefill = model.ops.stop_profile()
    dec = lambda p, rec=None: model.step([StepEntry(s, p, [rng.randrange(V)], [0]) for s in slots], record=rec)
    dec(prompt_len)
    rec = {}
    model.ops.start_profile()
    dec(prompt_len + 1, rec)
    decode = model.ops.stop_profile()
    distinct = [int(torch.unique(ids).numel()) for ids in rec.get("experts", [])]
    for s in slots:
        model.cache.release(s)
    model.use_graphs = graphs
    return prefill, decode, distinct


def graph_step_table(model, cfg, batch, prompt_len, rng):
    """The kernels of one captured decode step with the time each adds to the step: inside the graph, kernels
    start early under programmatic dependent launch and wait for the one before, so a kernel's share is the time
    from the end of the kernel before it to its own end (device timestamps of one replay, read through
    torch.profiler).  Kernels are named by pairing them, in order, with the launches of one eager step of the
    same shape.  Returns ({label: (launches, ms)}, distinct experts per layer) or None if the profiler is not
    available or the two sequences do not pair up."""
    import torch
    from flint_b200.engine.step import StepEntry
    try:
        from torch.profiler import ProfilerActivity, profile as torch_profile
    except ImportError:
        return None
    V = cfg["vocab_size"]
    slots = [model.cache.admit() for _ in range(batch)]
    for s in slots:
        model.cache.ensure(s, 0, prompt_len + 8)
        model.step([StepEntry(s, 0, [rng.randrange(V) for _ in range(prompt_len)], [])])
    pos = prompt_len

    def dec(rec=None):
        nonlocal pos
        out = model.step([StepEntry(s, pos, [rng.randrange(V)], [0]) for s in slots], record=rec)
        pos += 1
        return out
    graphs, model.use_graphs = model.use_graphs, False
    dec()
    rec = {}
    model.ops.start_profile()
    dec(rec)
    labels = [name for name, _ in model.ops.stop_profile(ordered=True)]
    distinct = [int(torch.unique(ids).numel()) for ids in rec.get("experts", [])]
    model.use_graphs = graphs
    table = None
    if graphs:
        for _ in range(3):
            dec()
        torch.cuda.synchronize()
        try:
            with torch_profile(activities=[ProfilerActivity.CUDA]) as prof:
                dec()
                torch.cuda.synchronize()
            ev = sorted(((e.time_range.start, e.time_range.end, e.name) for e in prof.events()
                         if e.device_type == torch.autograd.DeviceType.CUDA and "Memcpy" not in e.name and "Memset" not in e.name))
        except Exception:            # no CUPTI here: the caller falls back to the eager table
            ev = []
        followers = ("splitk_reduce", "attention_combine")      # second kernels of a launcher call
        paired, i = [], 0
        for start, end, name in ev:
            if any(f in name for f in followers) and paired:
                paired.append((paired[-1][0], end))
            elif i < len(labels):
                paired.append((labels[i], end))
                i += 1
            else:
                i += 1
        if ev and i == len(labels):
            table, prev = {}, ev[0][0]
            for label, end in paired:
                n, ms = table.get(label, (0, 0.0))
                table[label] = (n + 1, ms + max(0.0, end - prev) / 1000.0)
                prev = max(prev, end)
    for s in slots:
        model.cache.release(s)
    return (table, distinct) if table else None


def kernel_class(name, cfg):
    """The dominant kernels by what they compute; everything else is the small row-wise work."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    if "attention_prefill" in name:
        return "attention_prefill"
    if "attention" in name:
        return "attention_decode"
    if "gemm" in name and " " in name:
        shape = name.split(" ")[1]
        n, k = (int(x) for x in shape.split("x"))
        if "experts" in name:
            return "expert_gate_up" if k == H else "expert_down"
        if n == (nq + 2 * nkv) * hd and k == H:
            return "qkv"
        if n == V:
            return "head"
        if n == H and k == nq * hd:
            return "o_proj"
    return "other"


def kernel_fractions(table, cfg, pk, kind, n_tokens, kv_lens, distinct):
    """Flat {class.us, class.frac}: device time of each dominant kernel over a whole step and its fraction of the
    measured peak: bytes it must read over the copy bandwidth for a decode step, flops over the sustained library
    product rate for a prefill.  ``other`` (norms with routing, rotary write, plan, activation, embedding) has a
    time only."""
    H, I, L, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"], cfg["vocab_size"]
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    us = {}
    for name, (_, ms) in table.items():
        c = kernel_class(name, cfg)
        us[c] = us.get(c, 0.0) + ms * 1000.0
    keys = sum(kv_lens)
    if kind == "decode":
        work = {"qkv": L * (nq + 2 * nkv) * hd * H * 2, "o_proj": L * H * nq * hd * 2,
                "expert_gate_up": sum(distinct) * 2 * I * H * 2, "expert_down": sum(distinct) * H * I * 2,
                "attention_decode": keys * nkv * hd * 2 * 2 * L, "head": V * H * 2}
        peak = pk["hbm_gbs"] * 1e9
    else:
        T = n_tokens
        work = {"qkv": 2 * T * (nq + 2 * nkv) * hd * H * L, "o_proj": 2 * T * H * nq * hd * L,
                "expert_gate_up": 2 * (2 * T) * (2 * I) * H * L, "expert_down": 2 * (2 * T) * H * I * L,
                "attention_prefill": 4 * nq * hd * keys * L}
        peak = pk["bf16_tflops_sustained"] * 1e12
    out = {}
    for c, t in sorted(us.items(), key=lambda kv: -kv[1]):
        out[f"{kind}.{c}.us"] = round(t, 1)
        if c in work and t > 0:
            out[f"{kind}.{c}.frac"] = round(work[c] / (t * 1e-6) / peak, 3)
    return out


def profile(model, cfg, args, rng):
    """``--profile``: the tables to stderr."""
    prefill, decode, _ = profile_tables(model, cfg, args.batch, args.prompt_tokens, rng)

    def show(title, table):
        total = sum(ms for _, ms in table.values())
        print(f"--- {title}: {total:.3f} ms in {sum(n for n, _ in table.values())} launches", file=sys.stderr)
        for name, (n, ms) in sorted(table.items(), key=lambda kv: -kv[1][1]):
            print(f"{name:48s} {n:6d} launches {ms:10.3f} ms {100 * ms / total:6.1f} %", file=sys.stderr)
    show(f"prefill of {args.prompt_tokens} tokens", prefill)
    show(f"decode step, batch {args.batch}, context {args.prompt_tokens}", decode)
    return 0


def one_step(model, cfg, args, rng):
    """Set-up, one warm step and one more step of the asked kind, eagerly (no graph), for profilers."""
    import torch
    from flint_b200.engine.step import StepEntry
    V = cfg["vocab_size"]
    model.use_graphs = False
    n = args.prompt_tokens
    slots = [model.cache.admit() for _ in range(args.batch)]
    if args.one_step == "decode":
        for s in slots:
            model.cache.ensure(s, 0, n + 2)
            model.step([StepEntry(s, 0, [rng.randrange(V) for _ in range(n)], [])])
        step = lambda p: model.step([StepEntry(s, p, [rng.randrange(V)], [0]) for s in slots])
        step(n)
        torch.cuda.synchronize()
        before = model.ops.launches
        step(n + 1)
    else:
        run = lambda s: (model.cache.ensure(s, 0, n), model.step([StepEntry(s, 0, [rng.randrange(V) for _ in range(n)], [n - 1])]))
        run(slots[0])
        torch.cuda.synchronize()
        before = model.ops.launches
        run(slots[1 % len(slots)])
    torch.cuda.synchronize()
    print(f"launcher calls before the last step: {before}, in it: {model.ops.launches - before} "
          f"(a call with a split launches two kernels)", file=sys.stderr)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-tokens", type=int, default=2048)
    ap.add_argument("--ctx-size", type=int, default=4096)
    # the reference bench's own names for the sizes and the workload (crates/thuban_bench/src/main.rs:12-63)
    for flag in ("--hidden", "--intermediate", "--q-heads", "--kv-heads", "--head-dim", "--vocab", "--prefill-tokens",
                 "--decode-tokens", "--max-seq"):
        ap.add_argument(flag, type=int, default=None)
    ap.add_argument("--mixed", type=int, nargs=4, metavar=("REQUESTS", "MIN_PROMPT", "MAX_PROMPT", "DECODE"), default=None,
                    help="instead of the default run: continuous batching of this many requests through the engine")
    ap.add_argument("--expert-intermediate", type=int, default=None,
                    help="expert width (default 960, the Phi-mini-MoE sizes; 6400 gives the Phi-3.5-MoE sizes)")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (both are named)")
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--one-step", choices=["decode", "prefill"], default=None,
                    help="run the set-up, then one warm and one measured eager step of this kind, and exit "
                         "(for a launch list under ncu: the launch counts to skip and capture go to stderr)")
    ap.add_argument("--tiny", choices=["A", "B"], default=None,
                    help="instead of the default run: the tiny workload of that test configuration, in 32-bit, against "
                         "the timed CPU baseline (the plain C++ implementation)")
    ap.add_argument("--long", action="store_true",
                    help="instead of the default run: prompts of 4 x 32,768 and one of 130,944 tokens (with its 128 decoded "
                         "tokens the model's 131,072 positions) in portions of 2,048, then 128 decoded tokens each; "
                         "use with --expert-intermediate 6400 for the Phi-3.5-MoE sizes")
    ap.add_argument("--long-prompts", type=int, nargs="+", default=None, help="other prompt lengths for --long")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel table")
    ap.add_argument("--sweep", action="store_true",
                    help="instead of the default run: decode at batch 1 and 8 with contexts of 16,384 and 65,536 tokens, "
                         "batch 1 with 131,008, and batch 128 and 256 with 2,048, each with its roofline fraction")
    ap.add_argument("--profile", action="store_true",
                    help="print per-kernel device times of one prefill and one decode step to stderr and exit")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "formetaohy/Flint is a Rust workspace that reaches the GPU only through wgpu on Vulkan/Metal: "
                          "no Python package to install offline, no cargo here, no graphics API on this box"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(args.warmup, 3)

    import torch
    pk = peaks()
    cfg = mini_config(args.layers, args.expert_intermediate or args.intermediate,
                      {"hidden_size": args.hidden, "num_attention_heads": args.q_heads, "num_key_value_heads": args.kv_heads,
                       "head_dim": args.head_dim, "vocab_size": args.vocab})
    if args.max_seq:
        args.ctx_size = args.max_seq
    if args.prefill_tokens:
        args.prompt_tokens = args.prefill_tokens
    if args.decode_tokens:
        args.steps = args.decode_tokens
    rng = random.Random(0)
    if args.tiny:
        print(json.dumps(run_tiny(args.tiny)))
        return 0
    if args.sweep:
        print(json.dumps(run_sweep(cfg, pk, rng, max(8, args.steps // 4), warmup)))
        return 0
    if args.long:
        print(json.dumps(run_long(cfg, pk, rng, args.long_prompts or [32768] * 4 + [131072 - 128], 128)))
        return 0
    max_batch = max(args.batch, 1 if args.no_points else 64, args.mixed[0] if args.mixed else 1)
    model = build_model(cfg, max_batch, args.ctx_size)

    if args.profile:
        return profile(model, cfg, args, rng)
    if args.one_step:
        return one_step(model, cfg, args, rng)
    if args.mixed:
        n, lo, hi, dec = args.mixed
        for _ in range(2):          # the first pass compiles kernels and captures graphs
            r = run_mixed(model, cfg, n, lo, hi, dec, rng)
        print(json.dumps({"metric": f"mixed serving: {n} requests, prompts of {lo}..{hi} tokens, {dec} decoded each",
                          "value": round((r["prompt_tokens"] + r["decoded"]) / r["seconds"], 1), "unit": "tokens/s (prompt + decoded)",
                          "decode_tok_s": round(r["decoded"] / r["seconds"], 1), **r}))
        return 0

    clocks = ClockSampler()
    clocks.start()
    pre_ms = run_prefill(model, cfg, 2048, reps=3, warmup=3, rng=rng)
    dec = run_decode(model, cfg, args.batch, args.prompt_tokens, args.steps, warmup, rng)
    clock = clocks.stop()
    e2e = run_e2e(model, cfg, args.batch, args.prompt_tokens, args.steps, warmup, rng)
    points, points_frac = {}, {}
    if not args.no_points:
        for b in (1, 64):
            r = run_decode(model, cfg, b, args.prompt_tokens, max(8, args.steps // 2), warmup, rng)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
            # the same roofline as the headline's: bytes the step must read over its time, of the copy peak
            points_frac[f"decode_b{b}"] = round(decode_bytes(cfg, model, r["kv_lens"], r["distinct"]) / (r["ms"] * 1e-3) / 1e9
                                                / pk["hbm_gbs"], 4)

    kernels = {}
    kernels_decode_how = "CUDA events around every launch of one eager step (launches serialised, host gaps included)"
    if not args.no_kernels:
        pre_t, dec_t, distinct = profile_tables(model, cfg, args.batch, args.prompt_tokens, rng)
        in_graph = graph_step_table(model, cfg, args.batch, args.prompt_tokens, rng)
        if in_graph is not None:
            dec_t, distinct = in_graph
            kernels_decode_how = ("device timestamps of one replay of the captured step: a kernel's time runs from the end "
                                  "of the kernel before it to its own end (kernels overlap under programmatic dependent launch)")
        kernels.update(kernel_fractions(dec_t, cfg, pk, "decode", args.batch, [args.prompt_tokens + 2] * args.batch, distinct))
        kernels.update(kernel_fractions(pre_t, cfg, pk, "prefill", args.prompt_tokens, range(1, args.prompt_tokens + 1), None))
    pre_flops = step_flops(cfg, 2048, range(1, 2049))
    bytes_step = decode_bytes(cfg, model, dec["kv_lens"], dec["distinct"])
    achieved = bytes_step / (dec["ms"] * 1e-3) / 1e9
    mini = all(cfg[k] == MINI[k] for k in MINI if k != "num_hidden_layers")
    out = {
        "metric": f"decode tok/s at batch {args.batch} ({'Phi-mini-MoE layer sizes' if mini else 'other layer sizes, see config'}, "
                  f"{args.prompt_tokens:,}-token prompts, context {args.ctx_size:,})",
        "value": round(dec["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(dec["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights, uniform-random token ids", "impl": "ours",
        "config": config_of(cfg, args.batch, args.prompt_tokens, args.ctx_size, pk),
        "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tokens/s", "ms_per_step": round(e2e["ms"], 4),
                "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"]},
        "gpu_launches": dec["launches"],
        "prefill": {"value": round(2048 * 1000.0 / pre_ms, 1), "tokens": 2048, "ms": round(pre_ms, 3),
                    "frac": round(pre_flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                    "frac_of_sustained": round(pre_flops / (pre_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": bytes_step,
                     "distinct_experts_per_layer": round(sum(dec["distinct"]) / len(dec["distinct"]), 2)},
        "points": points,
        "points_roofline_frac": points_frac,
        "kernels": kernels,
        "kernels_how": "microseconds per step and fraction of the measured peak.  decode: " + kernels_decode_how +
                       "; fractions: bytes the kernel must read over the measured copy bandwidth.  prefill: CUDA events "
                       "around every launch of one eager step; fractions: flops over the measured sustained library "
                       "product rate",
        "clocks": clock,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
