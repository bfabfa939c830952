"""Each part alone on the GPU beside its plain function, and the generality of the composition:
a toy mixer with state of its own, a dense feed-forward, an RMS norm, a parallel block, a layer
that runs twice and a layer that reads another layer's cache; and a second toy model with a feed-forward
that routes by itself and a position encoding of its own -- all registered and built from the test,
without a change to the package."""
import math

import pytest
import torch

import plain_phimoe as P
from flint_b200.cache.manager import CacheManager, KVSpec, StateSpec
from flint_b200.config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from flint_b200.engine.model import Model
from flint_b200.engine.step import StepEntry, StepStaging
from flint_b200.parts.base import BuildContext, FeedForward, Mixer, PositionEncoding, mat
from flint_b200.registry import ARCHITECTURES, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS
from flint_b200.weights.sources import RandomSource

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ctx_for(dtype):
    from flint_b200.csrc.ops import get_ops
    return BuildContext(ops=get_ops(DEV), device=torch.device(DEV), compute=dtype)


def load_random(part, seed=0, dtype=torch.float32):
    src = RandomSource(part.weights(), seed, dtype=dtype)
    from flint_b200.weights.loader import place
    t = {n: place(src.read(n), ws, part.ctx.compute, DEV) for n, ws in part.weights().items()}
    part.load(t)
    return {n: v.double().cpu() for n, v in t.items()}


@pytest.mark.parametrize("kind,params", [("layernorm", {"width": 72, "eps": 1e-6, "bias": True}),
                                         ("layernorm", {"width": 100, "eps": 1e-5, "bias": False}),
                                         ("rmsnorm", {"width": 72, "eps": 1e-6})])
def test_norm_part(kind, params):
    part = NORMS.get(kind)(params, ctx_for("bfloat16"))
    w = load_random(part)
    x = torch.randn(9, params["width"]) * 2 + 0.5
    out = part.forward(x.to(DEV), (torch.float32, torch.bfloat16))
    if kind == "layernorm":
        exp = P.layer_norm(x.double(), w["weight"], w.get("bias"), params["eps"])
    else:
        exp = x.double() / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + params["eps"]) * w["weight"]
    assert (out[torch.float32].double().cpu() - exp).abs().max() < 1e-5
    assert (out[torch.bfloat16].double().cpu() - exp).abs().max() < 3e-2


def test_rope_part_tables():
    cfg = {"rope_theta": 500000.0, "max_position_embeddings": 512, "original_max_position_embeddings": 64,
           "rope_scaling": {"type": "longrope", "short_factor": [1.0 + 0.1 * i for i in range(16)],
                            "long_factor": [2.0 + 0.1 * i for i in range(16)], "short_mscale": 1.1, "long_mscale": 1.3}}
    part = POSITION_ENCODINGS.get("rope")({"rotary_dim": 32, "theta": 500000.0, "max_positions": 512,
                                           "short_factor": cfg["rope_scaling"]["short_factor"],
                                           "long_factor": cfg["rope_scaling"]["long_factor"],
                                           "original_max_positions": 64, "short_mscale": 1.1, "long_mscale": 1.3},
                                          ctx_for("float32"))
    cos, sin = part.tables()
    ec, es = P.rope_tables(cfg, 32, 512)
    assert (cos.double().cpu() - ec).abs().max() < 1e-6 and (sin.double().cpu() - es).abs().max() < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_part_alone(dtype):
    """The attention mixer with a cache of its own, in two portions, beside the plain functions."""
    H, nq, nkv, hd, T = 80, 5, 5, 16, 50
    rope = PartSpec("rope", {"rotary_dim": 8, "theta": 10000.0, "max_positions": 128})
    ctx = ctx_for(dtype)
    part = MIXERS.get("attention")({"hidden_size": H, "num_heads": nq, "num_kv_heads": nkv, "head_dim": hd, "window": 20,
                                    "qkv_bias": True, "out_bias": True, "position": rope}, ctx)
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    w = load_random(part, dtype=store)
    cm = CacheManager({0: part.cache_spec()}, {}, page_size=16, n_pages=8, max_slots=2, max_context=128,
                      dtype=store, device=DEV)
    slot = cm.admit()
    x = torch.randn(T, H)
    staging = StepStaging(64, DEV, needs=[part.step_needs()])
    res = torch.zeros(T, H, device=DEV)
    for a, b in ((0, 33), (33, 50)):
        cm.ensure(slot, a, b)
        cm.sync()
        step = staging.pack([StepEntry(slot, a, [0] * (b - a), [])], 10, 128)
        xin = {dt: x[a:b].to(DEV).to(dt) for dt in part.input_dtypes()}
        pend = part.forward(xin, res[a:b], step, cm.view(0), None)
        ctx.ops.apply_pending(res[a:b], pend)        # the output projection is left pending for the next norm
        cm.advance(slot, b)
    xd = x.double() if dtype == "float32" else x.to(torch.bfloat16).double()
    cos, sin = P.rope_tables({"rope_theta": 10000.0, "partial_rotary_factor": 0.5}, hd, T)
    q = P.rope_rotate(P.linear(xd, w["q_proj.weight"], w["q_proj.bias"]).view(T, nq, hd), cos, sin)
    k = P.rope_rotate(P.linear(xd, w["k_proj.weight"], w["k_proj.bias"]).view(T, nkv, hd), cos, sin)
    v = P.linear(xd, w["v_proj.weight"], w["v_proj.bias"]).view(T, nkv, hd)
    exp = P.linear(P.attention(q, k, v, 20).reshape(T, nq * hd), w["o_proj.weight"], w["o_proj.bias"])
    tol = 1e-5 if dtype == "float32" else 2e-2 * float(exp.abs().max())
    assert (res.double().cpu() - exp).abs().max() < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["sparsemixer_moe", "gated_mlp"])
def test_feed_forward_parts_alone(kind, dtype):
    H, I, E, T = 72, 40, 5, 37
    ctx = ctx_for(dtype)
    params = {"hidden_size": H, "intermediate_size": I, "act": "silu"}
    if kind == "sparsemixer_moe":
        params.update(num_experts=E, jitter_eps=0.05)
    part = FEED_FORWARDS.get(kind)(params, ctx)
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    w = load_random(part, dtype=store)
    x = torch.randn(T, H)
    xin = {dt: x.to(DEV).to(dt) for dt in part.input_dtypes()}
    res = torch.zeros(T, H, device=DEV)
    step = type("S", (), {"record": {}})()
    pend = part.forward(xin, res, step)
    if pend is not None:                              # the experts' gated sum is left pending
        ctx.ops.apply_pending(res, pend)
    x64 = x.double()
    xa = x64 if dtype == "float32" else x.to(torch.bfloat16).double()
    if kind == "gated_mlp":
        exp = P.expert_mlp(xa, w["gate_proj.weight"], w["up_proj.weight"], w["down_proj.weight"])
    else:
        exp = torch.zeros(T, H, dtype=torch.float64)
        logits = x64 @ w["gate.weight"].T
        chosen = []
        for t in range(T):
            i1, g1, i2, g2 = P.sparsemixer_top2(logits[t], 0.05)
            chosen.append([i1, i2])
            ex = lambda e: P.expert_mlp(xa[t:t + 1], w[f"experts.{e}.w1.weight"], w[f"experts.{e}.w3.weight"], w[f"experts.{e}.w2.weight"])[0]
            exp[t] = g1 * ex(i1) + g2 * ex(i2)
        assert step.record["experts"][0].cpu().tolist() == chosen       # the same experts, first
    tol = 1e-5 if dtype == "float32" else 3e-2 * float(exp.abs().max())
    assert (res.double().cpu() - exp).abs().max() < tol


# ------------------------------------------------------------------------------------------------
# a toy architecture defined here: a mixer with state of its own, parts the engine's model does not use

class RunningSumMixer(Mixer):
    """out[t] = W (state + x[first..t] summed) * 0.1; the state is the running sum of the request."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.width = params["width"]

    def weights(self):
        return {"mix.weight": mat(self.width, self.width)}

    def load(self, t):
        self.w = t["mix.weight"].float()

    def input_dtypes(self):
        return (torch.float32,)

    def state_spec(self):
        return StateSpec((self.width,), torch.float32)

    def forward(self, x, residual, step, cache, state, writes_cache=True):
        x32 = x[torch.float32]
        for e, row0 in zip(step.entries, step.entry_start):
            n = len(e.tokens)
            run = state[e.slot] + torch.cumsum(x32[row0:row0 + n], 0)
            residual[row0:row0 + n] += (run @ self.w.T) * 0.1
            state[e.slot] = run[-1]


def toy_spec(H=48, V=97):
    rope = PartSpec("rope", {"rotary_dim": 16, "theta": 10000.0, "max_positions": 256})
    attn = PartSpec("attention", {"hidden_size": H, "num_heads": 3, "num_kv_heads": 3, "head_dim": 16, "window": 0,
                                  "qkv_bias": False, "out_bias": False, "position": rope})
    rms = PartSpec("rmsnorm", {"width": H, "eps": 1e-6})
    ln = PartSpec("layernorm", {"width": H, "eps": 1e-5, "bias": True})
    mlp = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": 64, "act": "gelu_pytorch_tanh"})
    toy = PartSpec("test_running_sum", {"width": H})
    names = {"norm1": "n1.", "mixer": "mix.", "norm2": "n2.", "ffn": "ff."}
    layers = (LayerSpec("prenorm", {"norm1": rms, "mixer": toy, "norm2": rms, "ffn": mlp}, "layers.0.", names),
              LayerSpec("parallel", {"norm1": ln, "mixer": attn, "ffn": mlp}, "layers.1.", names),
              LayerSpec("prenorm", {"norm1": ln, "mixer": attn, "norm2": rms, "ffn": mlp}, "layers.2.", names))
    # layer 0 runs twice (shared weights, separate state); the last call reads the cache of call 1
    order = (LayerCall(0), LayerCall(1), LayerCall(0), LayerCall(2, cache_of=1))
    return ModelSpec(architecture="ToyStateLM", vocab_size=V, hidden_size=H, max_positions=256, layers=layers,
                     order=order, final_norm=rms, head_bias=False, tie_word_embeddings=True)


def toy_plain(spec, w, tokens):
    """Whole-sequence computation of the toy model with the plain functions."""
    T = len(tokens)
    h = P.embed(tokens, w["embed_tokens.weight"])
    rms = lambda x, g: x / torch.sqrt((x ** 2).mean(-1, keepdim=True) + 1e-6) * g
    mlp = lambda x, p: (P.activation(x @ w[p + "gate_proj.weight"].T, "gelu_pytorch_tanh") * (x @ w[p + "up_proj.weight"].T)) @ w[p + "down_proj.weight"].T
    cos, sin = P.rope_tables({"rope_theta": 10000.0}, 16, T)
    kv1 = None
    for call in spec.order:
        p = f"layers.{call.layer}."
        if call.layer == 0:
            x = rms(h, w[p + "n1.weight"])
            h = h + (torch.cumsum(x, 0) @ w[p + "mix.mix.weight"].T) * 0.1
            h = h + mlp(rms(h, w[p + "n2.weight"]), p + "ff.")
            continue
        x = P.layer_norm(h, w[p + "n1.weight"], w[p + "n1.bias"], 1e-5)
        q = P.rope_rotate((x @ w[p + "mix.q_proj.weight"].T).view(T, 3, 16), cos, sin)
        if call.cache_of is None:
            k = P.rope_rotate((x @ w[p + "mix.k_proj.weight"].T).view(T, 3, 16), cos, sin)
            v = (x @ w[p + "mix.v_proj.weight"].T).view(T, 3, 16)
            kv1 = (k, v)
        a = P.attention(q, kv1[0], kv1[1], 0).reshape(T, 48) @ w[p + "mix.o_proj.weight"].T
        if call.layer == 1:               # parallel block: both read the same normed input
            h = h + a + mlp(x, p + "ff.")
        else:
            h = h + a
            h = h + mlp(rms(h, w[p + "n2.weight"]), p + "ff.")
    return rms(h, w["norm.weight"]) @ w["embed_tokens.weight"].T


def test_toy_architecture_with_a_stateful_mixer_is_built_and_stepped():
    MIXERS.register("test_running_sum", RunningSumMixer, replace=True)

    class ToyArch:
        @staticmethod
        def parse_config(d):
            return d

        @staticmethod
        def model_spec(cfg):
            return toy_spec()
    ARCHITECTURES.register("ToyStateLM", ToyArch, replace=True)
    try:
        from flint_b200.engine.model import architecture_of
        spec = architecture_of({"architectures": ["ToyStateLM"]}).model_spec({})
        from flint_b200.engine.model import Layer, expected_tensors
        expected = expected_tensors(spec, [Layer(ls, ctx_for("float32")) for ls in spec.layers],
                                    NORMS.get(spec.final_norm.kind)(spec.final_norm.params, ctx_for("float32")))
        src = RandomSource(expected, 3, dtype=torch.float32)
        model = Model(spec, src, dtype="float32", device=DEV, page_size=16, n_pages=12, max_slots=3)
        assert sorted(model.cache.state) == [0, 2] and len(model.cache.groups) == 1
        assert model.cache.groups[0].calls == [1]          # call 3 reads call 1's cache and owns none
        w = {n: src.read(n).double() for n in expected}
        seqs = {0: [i * 7 % 97 for i in range(60)], 1: [i * 11 % 97 for i in range(41)]}
        want = {k: toy_plain(spec, w, t) for k, t in seqs.items()}
        # two requests side by side, in portions of changing size, one decoded token by token at the end
        slots = {k: model.cache.admit() for k in seqs}
        done = {k: 0 for k in seqs}
        got = {k: [] for k in seqs}
        sizes = [5, 2, 9, 1, 1, 17, 3, 1, 30, 64]
        i = 0
        while any(done[k] < len(seqs[k]) for k in seqs):
            entries, ks = [], []
            for k in seqs:
                n = min(sizes[(i + k) % len(sizes)], len(seqs[k]) - done[k])
                if n <= 0:
                    continue
                model.cache.ensure(slots[k], done[k], done[k] + n)
                entries.append(StepEntry(slots[k], done[k], seqs[k][done[k]:done[k] + n], list(range(n))))
                ks.append((k, n))
            out = model.step(entries).cpu()
            r = 0
            for k, n in ks:
                got[k].append(out[r:r + n])
                r += n
                done[k] += n
            i += 1
        for k in seqs:
            err = (torch.cat(got[k]).double() - want[k]).abs().max().item()
            assert err < 1e-4, f"request {k}: {err:.2e}"
        # a slot that is used again starts from zero state
        model.cache.release(slots[0])
        s = model.cache.admit()
        model.cache.ensure(s, 0, 10)
        again = model.step([StepEntry(s, 0, seqs[0][:10], list(range(10)))]).cpu()
        assert (again.double() - want[0][:10]).abs().max().item() < 1e-4
    finally:
        MIXERS.unregister("test_running_sum")
        ARCHITECTURES.unregister("ToyStateLM")


# ------------------------------------------------------------------------------------------------
# a second toy architecture: a feed-forward with routing of its own and another position encoding

class SwitchFeedForward(FeedForward):
    """Top-1 routing over small ReLU experts: y = p_e * W2_e relu(W1_e x), e = argmax of the router logits,
    p = softmax(logits)[e].  Written with ordinary tensor operations: a part may compute however it likes."""

    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.width, self.inner, self.experts = params["width"], params["inner"], params["experts"]

    def weights(self):
        return {"router.weight": mat(self.experts, self.width), "w1.weight": mat(self.experts * self.inner, self.width),
                "w2.weight": mat(self.experts * self.width, self.inner)}

    def load(self, t):
        self.wr = t["router.weight"].float()
        self.w1 = t["w1.weight"].float().view(self.experts, self.inner, self.width)
        self.w2 = t["w2.weight"].float().view(self.experts, self.width, self.inner)

    def input_dtypes(self):
        return (torch.float32,)

    def forward(self, x, residual, step):
        x32 = x[torch.float32]
        prob = torch.softmax(x32 @ self.wr.T, -1)
        e = prob.argmax(-1)
        hid = torch.relu(torch.einsum("tw,tiw->ti", x32, self.w1[e]))
        residual += torch.einsum("ti,twi->tw", hid, self.w2[e]) * prob.gather(1, e[:, None])


class InterpolatedRotary(PositionEncoding):
    """Rotary angles of position / factor (position interpolation) over the first ``rotary_dim`` dims of a head."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.rotary_dim = int(params["rotary_dim"])

    def tables(self):
        half = self.rotary_dim // 2
        inv = float(self.params["theta"]) ** (-2.0 * torch.arange(half, dtype=torch.float64) / self.rotary_dim)
        ang = (torch.arange(int(self.params["max_positions"]), dtype=torch.float64) / float(self.params["factor"]))[:, None] * inv
        return torch.cos(ang).float().to(self.ctx.device), torch.sin(ang).float().to(self.ctx.device)


def routed_spec(H=40, V=61):
    pos = PartSpec("test_interpolated_rotary", {"rotary_dim": 8, "theta": 100.0, "factor": 3.5, "max_positions": 128})
    attn = PartSpec("attention", {"hidden_size": H, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16, "window": 24,
                                  "qkv_bias": True, "out_bias": False, "position": pos})
    ln = PartSpec("layernorm", {"width": H, "eps": 1e-5, "bias": True})
    switch = PartSpec("test_switch_ffn", {"width": H, "inner": 24, "experts": 5})
    names = {"norm1": "n1.", "mixer": "mix.", "norm2": "n2.", "ffn": "ff."}
    layers = tuple(LayerSpec("prenorm", {"norm1": ln, "mixer": attn, "norm2": ln, "ffn": switch}, f"layers.{i}.", names)
                   for i in range(2))
    return ModelSpec(architecture="ToyRoutedLM", vocab_size=V, hidden_size=H, max_positions=128, layers=layers,
                     order=(LayerCall(0), LayerCall(1)), final_norm=ln, head_bias=False, tie_word_embeddings=True)


def routed_plain(w, tokens):
    T = len(tokens)
    h = P.embed(tokens, w["embed_tokens.weight"])
    half = 4
    inv = 100.0 ** (-2.0 * torch.arange(half, dtype=torch.float64) / 8)
    ang = (torch.arange(T, dtype=torch.float64) / 3.5)[:, None] * inv
    cos, sin = torch.cos(ang), torch.sin(ang)
    for i in range(2):
        p = f"layers.{i}."
        x = P.layer_norm(h, w[p + "n1.weight"], w[p + "n1.bias"], 1e-5)
        q = P.rope_rotate((x @ w[p + "mix.q_proj.weight"].T + w[p + "mix.q_proj.bias"]).view(T, 4, 16), cos, sin)
        k = P.rope_rotate((x @ w[p + "mix.k_proj.weight"].T + w[p + "mix.k_proj.bias"]).view(T, 2, 16), cos, sin)
        v = (x @ w[p + "mix.v_proj.weight"].T + w[p + "mix.v_proj.bias"]).view(T, 2, 16)
        h = h + P.attention(q, k, v, 24).reshape(T, 64) @ w[p + "mix.o_proj.weight"].T
        x = P.layer_norm(h, w[p + "n2.weight"], w[p + "n2.bias"], 1e-5)
        prob = torch.softmax(x @ w[p + "ff.router.weight"].T, -1)
        e = prob.argmax(-1)
        w1, w2 = w[p + "ff.w1.weight"].view(5, 24, 40), w[p + "ff.w2.weight"].view(5, 40, 24)
        for t in range(T):
            h[t] = h[t] + (w2[e[t]] @ torch.relu(w1[e[t]] @ x[t])) * prob[t, e[t]]
    return P.layer_norm(h, w["norm.weight"], w["norm.bias"], 1e-5) @ w["embed_tokens.weight"].T


def test_toy_architecture_with_its_own_routing_and_position_encoding():
    """A feed-forward with routing and a position encoding that the package does not have, registered from here,
    built by the generic model and stepped in portions and token by token (one-token batches go through the
    graph path, which the toy feed-forward declares itself safe for)."""
    FEED_FORWARDS.register("test_switch_ffn", SwitchFeedForward, replace=True)
    POSITION_ENCODINGS.register("test_interpolated_rotary", InterpolatedRotary, replace=True)

    class RoutedArch:
        @staticmethod
        def parse_config(d):
            return d

        @staticmethod
        def model_spec(cfg):
            return routed_spec()
    ARCHITECTURES.register("ToyRoutedLM", RoutedArch, replace=True)
    try:
        from flint_b200.engine.model import Layer, architecture_of, expected_tensors
        spec = architecture_of({"architectures": ["ToyRoutedLM"]}).model_spec({})
        expected = expected_tensors(spec, [Layer(ls, ctx_for("float32")) for ls in spec.layers],
                                    NORMS.get(spec.final_norm.kind)(spec.final_norm.params, ctx_for("float32")))
        src = RandomSource(expected, 5, dtype=torch.float32)
        model = Model(spec, src, dtype="float32", device=DEV, page_size=16, n_pages=8, max_slots=2)
        w = {n: src.read(n).double() for n in expected}
        tokens = [(i * 13 + 5) % 61 for i in range(70)]          # longer than the window of 24 and than 4 pages hold
        want = routed_plain(w, tokens)
        slot = model.cache.admit()
        got, done = [], 0
        for n in [9, 2, 17, 1, 1, 1, 30, 1, 1, 1, 1, 1, 1, 1, 1]:
            n = min(n, len(tokens) - done)
            if n <= 0:
                break
            model.cache.ensure(slot, done, done + n)
            got.append(model.step([StepEntry(slot, done, tokens[done:done + n], list(range(n)))]).cpu())
            done += n
            model.cache.advance(slot, done)
        err = (torch.cat(got).double() - want[:done]).abs().max().item()
        assert err < 1e-4, f"{err:.2e}"
        assert model.cache.groups[0].pages.pool.used_pages <= 3      # the window of 24 lets earlier pages go
    finally:
        FEED_FORWARDS.unregister("test_switch_ffn")
        POSITION_ENCODINGS.unregister("test_interpolated_rotary")
        ARCHITECTURES.unregister("ToyRoutedLM")


def test_a_stateful_mixer_is_recomputed_from_zero_after_preemption():
    """The toy model with the running-sum mixer through ``Engine`` with so few pages that requests are preempted
    and later recomputed from their prompt and generated tokens: the mixer's state slab must start from zero on
    every re-admission, or the recomputed tokens differ from the plain whole-sequence result."""
    from flint_b200.engine.engine import Engine
    from flint_b200.sampling.params import SamplingParams
    MIXERS.register("test_running_sum", RunningSumMixer, replace=True)
    try:
        from flint_b200.engine.model import Layer, expected_tensors
        spec = toy_spec()
        expected = expected_tensors(spec, [Layer(ls, ctx_for("float32")) for ls in spec.layers],
                                    NORMS.get(spec.final_norm.kind)(spec.final_norm.params, ctx_for("float32")))
        src = RandomSource(expected, 3, dtype=torch.float32)
        w = {n: src.read(n).double() for n in expected}
        prompts = [[(i * 7 + 3 * k) % 97 for i in range(n)] for k, n in enumerate((21, 30, 26))]
        preempted = 0
        for n_pages in (12, 5):
            model = Model(spec, src, dtype="float32", device=DEV, page_size=16, n_pages=n_pages, max_slots=3,
                          max_step_tokens=32)
            eng = Engine(model, SamplingParams.greedy(), prefill_chunk=16, stop=())
            got = eng.generate(prompts, 14)
            preempted += eng.scheduler.preemptions
            for p, g in zip(prompts, got):
                assert len(g) == 14
                logits = toy_plain(spec, w, list(p) + g)
                for j, tok in enumerate(g):
                    row = logits[len(p) - 1 + j]
                    best = int(torch.argmax(row))
                    assert tok == best or float(row[best] - row[tok]) < 1e-5, (n_pages, j, tok, best)
            assert model.cache.free_slots == 3
        assert preempted > 0, "pages never ran out"
    finally:
        MIXERS.unregister("test_running_sum")


# ------------------------------------------------------------------------------------------------
# a third toy architecture: positions added to the embedding, a rotation of neighbouring dims, and a mixer whose
# values are wider than its keys

class LearnedPositions(PositionEncoding):
    """h[t] += table[position of row t]: a position encoding that acts on the embedded rows."""

    graph_safe = True

    def weights(self):
        return {"weight": mat(int(self.params["max_positions"]), int(self.params["width"]))}

    def load(self, t):
        self.table = t["weight"].float()

    def after_embedding(self, h, step):
        h += self.table[step.pos.long()]


class NeighbourRotary(PositionEncoding):
    """Plain rotary angles, but dims 2i and 2i + 1 of a head rotate together."""
    style = "interleaved"

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.rotary_dim = int(params["rotary_dim"])

    def tables(self):
        half = self.rotary_dim // 2
        inv = float(self.params["theta"]) ** (-2.0 * torch.arange(half, dtype=torch.float64) / self.rotary_dim)
        ang = torch.arange(int(self.params["max_positions"]), dtype=torch.float64)[:, None] * inv
        return torch.cos(ang).float().to(self.ctx.device), torch.sin(ang).float().to(self.ctx.device)


class WideValueMixer(Mixer):
    """Causal attention with keys of 16 numbers and values of 24, written with ordinary tensor operations over
    the pages the cache manager gives it."""
    KD, VD, HEADS = 16, 24, 2

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.width = params["width"]

    def weights(self):
        n = self.HEADS
        return {"q.weight": mat(n * self.KD, self.width), "k.weight": mat(n * self.KD, self.width),
                "v.weight": mat(n * self.VD, self.width), "o.weight": mat(self.width, n * self.VD)}

    def load(self, t):
        self.w = {k: v.float() for k, v in t.items()}

    def input_dtypes(self):
        return (torch.float32,)

    def cache_spec(self):
        return KVSpec(self.HEADS, self.KD, 0, value_dim=self.VD)

    def forward(self, x, residual, step, cache, state, writes_cache=True):
        x32, n, P = x[torch.float32], self.HEADS, cache.page_size
        assert tuple(cache.k.shape[1:]) == (n, P, self.KD) and tuple(cache.v.shape[1:]) == (n, P, self.VD)
        q = (x32 @ self.w["q.weight"].T).view(-1, n, self.KD)
        k = (x32 @ self.w["k.weight"].T).view(-1, n, self.KD)
        v = (x32 @ self.w["v.weight"].T).view(-1, n, self.VD)
        pos, slot = step.pos.long(), step.slot.long()
        pages = cache.block_table[slot, pos // P].long()
        cache.k[pages, :, pos % P] = k.to(cache.k.dtype)
        cache.v[pages, :, pos % P] = v.to(cache.v.dtype)
        out = torch.zeros((x32.shape[0], n * self.VD), device=x32.device)
        for e, row0 in zip(step.entries, step.entry_start):
            js = torch.arange(e.start_pos + len(e.tokens), device=x32.device)
            pg = cache.block_table[e.slot, js // P].long()
            ks, vs = cache.k[pg, :, js % P].float(), cache.v[pg, :, js % P].float()      # [keys, heads, dim]
            for r in range(len(e.tokens)):
                seen = e.start_pos + r + 1
                s = torch.einsum("hd,khd->hk", q[row0 + r], ks[:seen]) / math.sqrt(self.KD)
                out[row0 + r] = torch.einsum("hk,khd->hd", torch.softmax(s, -1), vs[:seen]).reshape(-1)
        residual += out @ self.w["o.weight"].T


def wide_spec(H=40, V=53):
    rot = PartSpec("test_neighbour_rotary", {"rotary_dim": 8, "theta": 50.0, "max_positions": 96})
    attn = PartSpec("attention", {"hidden_size": H, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16, "window": 0,
                                  "qkv_bias": False, "out_bias": False, "position": rot})
    wide = PartSpec("test_wide_value", {"width": H})
    ln = PartSpec("layernorm", {"width": H, "eps": 1e-5, "bias": True})
    mlp = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": 32, "act": "silu"})
    names = {"norm1": "n1.", "mixer": "mix.", "norm2": "n2.", "ffn": "ff."}
    layers = (LayerSpec("prenorm", {"norm1": ln, "mixer": attn, "norm2": ln, "ffn": mlp}, "layers.0.", names),
              LayerSpec("prenorm", {"norm1": ln, "mixer": wide, "norm2": ln, "ffn": mlp}, "layers.1.", names))
    return ModelSpec(architecture="ToyWideLM", vocab_size=V, hidden_size=H, max_positions=96, layers=layers,
                     order=(LayerCall(0), LayerCall(1)), final_norm=ln, head_bias=False, tie_word_embeddings=True,
                     embed_position=PartSpec("test_learned_positions", {"max_positions": 96, "width": H}))


def wide_plain(w, tokens):
    T = len(tokens)
    h = P.embed(tokens, w["embed_tokens.weight"]) + w["embed_positions.weight"][:T]
    mlp = lambda x, p: P.expert_mlp(x, w[p + "gate_proj.weight"], w[p + "up_proj.weight"], w[p + "down_proj.weight"])
    inv = 50.0 ** (-2.0 * torch.arange(4, dtype=torch.float64) / 8)
    ang = torch.arange(T, dtype=torch.float64)[:, None] * inv
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

    def rotate(x):                      # dims 2i and 2i + 1 of the first 8 dims of a head
        a, b = x[..., 0:8:2], x[..., 1:8:2]
        both = torch.stack([a * cos - b * sin, b * cos + a * sin], -1).reshape(*x.shape[:-1], 8)
        return torch.cat([both, x[..., 8:]], -1)
    p = "layers.0."
    x = P.layer_norm(h, w[p + "n1.weight"], w[p + "n1.bias"], 1e-5)
    q = rotate((x @ w[p + "mix.q_proj.weight"].T).view(T, 4, 16))
    k = rotate((x @ w[p + "mix.k_proj.weight"].T).view(T, 2, 16))
    v = (x @ w[p + "mix.v_proj.weight"].T).view(T, 2, 16)
    h = h + P.attention(q, k, v, 0).reshape(T, 64) @ w[p + "mix.o_proj.weight"].T
    h = h + mlp(P.layer_norm(h, w[p + "n2.weight"], w[p + "n2.bias"], 1e-5), p + "ff.")
    p = "layers.1."
    x = P.layer_norm(h, w[p + "n1.weight"], w[p + "n1.bias"], 1e-5)
    q = (x @ w[p + "mix.q.weight"].T).view(T, 2, 16)
    k = (x @ w[p + "mix.k.weight"].T).view(T, 2, 16)
    v = (x @ w[p + "mix.v.weight"].T).view(T, 2, 24)
    a = torch.zeros(T, 2, 24, dtype=torch.float64)
    for t in range(T):
        s = torch.einsum("hd,khd->hk", q[t], k[:t + 1]) / 4.0
        a[t] = torch.einsum("hk,khd->hd", torch.softmax(s, -1), v[:t + 1])
    h = h + a.reshape(T, 48) @ w[p + "mix.o.weight"].T
    h = h + mlp(P.layer_norm(h, w[p + "n2.weight"], w[p + "n2.bias"], 1e-5), p + "ff.")
    return P.layer_norm(h, w["norm.weight"], w["norm.bias"], 1e-5) @ w["embed_tokens.weight"].T


def test_toy_architecture_with_embedded_positions_neighbour_rotation_and_wide_values():
    """Positions added to the embedding through the spec's hook, the package's attention with a position
    encoding of the other rotation style, and a mixer whose cached values are wider than its keys (a cache group
    of its own): registered and built from here, stepped in portions and token by token."""
    POSITION_ENCODINGS.register("test_learned_positions", LearnedPositions, replace=True)
    POSITION_ENCODINGS.register("test_neighbour_rotary", NeighbourRotary, replace=True)
    MIXERS.register("test_wide_value", WideValueMixer, replace=True)
    try:
        from flint_b200.engine.model import Layer, expected_tensors
        spec = wide_spec()
        c = ctx_for("float32")
        expected = expected_tensors(spec, [Layer(ls, c) for ls in spec.layers],
                                    NORMS.get(spec.final_norm.kind)(spec.final_norm.params, c),
                                    POSITION_ENCODINGS.get(spec.embed_position.kind)(spec.embed_position.params, c))
        assert "embed_positions.weight" in expected
        src = RandomSource(expected, 8, dtype=torch.float32)
        model = Model(spec, src, dtype="float32", device=DEV, page_size=16, n_pages=8, max_slots=2)
        assert len(model.cache.groups) == 2                     # keys of 16 with values of 16, and with values of 24
        assert {g.spec.value_width for g in model.cache.groups} == {16, 24}
        w = {n: src.read(n).double() for n in expected}
        tokens = [(i * 5 + 2) % 53 for i in range(60)]
        want = wide_plain(w, tokens)
        slot = model.cache.admit()
        got, done = [], 0
        for n in [7, 2, 19, 1, 1, 25, 1, 1, 1, 1, 1]:
            n = min(n, len(tokens) - done)
            model.cache.ensure(slot, done, done + n)
            got.append(model.step([StepEntry(slot, done, tokens[done:done + n], list(range(n)))]).cpu())
            done += n
            model.cache.advance(slot, done)
        err = (torch.cat(got).double() - want[:done]).abs().max().item()
        assert err < 1e-4, f"{err:.2e}"
    finally:
        POSITION_ENCODINGS.unregister("test_learned_positions")
        POSITION_ENCODINGS.unregister("test_neighbour_rotary")
        MIXERS.unregister("test_wide_value")
