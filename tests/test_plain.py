"""The plain implementation pinned to values worked out by hand (the reference pins its CPU twins
the same way: crates/thuban_backend/tests/kernels.rs:1310-1481), and the host sampler."""
import math

import numpy as np
import pytest
import torch

import plain_phimoe
import plain_phimoe as P

D = torch.float64


def test_layer_norm_by_hand():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=D)          # mean 3, var (4+1+0+9)/4 = 3.5
    y = P.layer_norm(x, torch.tensor([1.0, 2.0, 1.0, 0.5], dtype=D), torch.tensor([0.0, 1.0, 0.0, -1.0], dtype=D), 0.0)
    r = 1 / math.sqrt(3.5)
    assert torch.allclose(y, torch.tensor([[-2 * r, -2 * r + 1, 0.0, 1.5 * r - 1]], dtype=D))


def test_linear_by_hand():
    x = torch.tensor([[1.0, 2.0], [3.0, 4.0]], dtype=D)
    w = torch.tensor([[5.0, 6.0], [7.0, 8.0]], dtype=D)          # y = x W^T
    assert P.linear(x, w).tolist() == [[17.0, 23.0], [39.0, 53.0]]
    assert P.linear(x, w, torch.tensor([1.0, -1.0], dtype=D)).tolist() == [[18.0, 22.0], [40.0, 52.0]]


def test_rope_with_longrope_factor_and_scale_by_hand():
    cfg = {"rope_theta": 100.0, "max_position_embeddings": 16, "original_max_position_embeddings": 4,
           "rope_scaling": {"type": "longrope", "short_factor": [1.0, 2.0], "long_factor": [4.0, 1.0]}}
    cos, sin = P.rope_tables(cfg, 4, 6)
    m = math.sqrt(1 + math.log(16 / 4) / math.log(4))            # sqrt(2)
    # position 1 (short): inv = [1, 100^(-1/2)] / [1, 2] = [1, 0.05]
    assert torch.allclose(cos[1], torch.tensor([math.cos(1.0), math.cos(0.05)], dtype=D) * m)
    # position 5 (long): inv = [1/4, 0.1]
    assert torch.allclose(sin[5], torch.tensor([math.sin(1.25), math.sin(0.5)], dtype=D) * m)
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]], dtype=D)          # half-split pairs (1,3) and (2,4)
    y = P.rope_rotate(x, cos[1:2], sin[1:2])
    c0, s0, c1, s1 = cos[1, 0], sin[1, 0], cos[1, 1], sin[1, 1]
    assert torch.allclose(y[0, 0], torch.stack([1 * c0 - 3 * s0, 2 * c1 - 4 * s1, 3 * c0 + 1 * s0, 4 * c1 + 2 * s1]))
    # no scaling: plain table, no scale
    cos2, _ = P.rope_tables({"rope_theta": 100.0}, 4, 3)
    assert torch.allclose(cos2[2], torch.tensor([math.cos(2.0), math.cos(0.2)], dtype=D))
    # partial rotary: dims beyond the rotary part pass through
    z = P.rope_rotate(torch.tensor([[[1.0, 2.0, 9.0, 8.0]]], dtype=D), cos[1:2, :1], sin[1:2, :1])
    assert z[0, 0, 2:].tolist() == [9.0, 8.0]


def test_attention_causal_and_window_by_hand():
    # one head, head size 1, scale 1: scores are q*k
    q = torch.tensor([[[0.0]], [[1.0]], [[1.0]]], dtype=D)
    k = torch.tensor([[[1.0]], [[2.0]], [[0.0]]], dtype=D)
    v = torch.tensor([[[10.0]], [[20.0]], [[30.0]]], dtype=D)
    o = P.attention(q, k, v, 0)
    assert abs(o[0, 0, 0].item() - 10.0) < 1e-12                                     # only itself
    w = math.exp(1) / (math.exp(1) + math.exp(2))
    assert abs(o[1, 0, 0].item() - (10 * w + 20 * (1 - w))) < 1e-12
    e = [math.exp(1), math.exp(2), math.exp(0)]
    assert abs(o[2, 0, 0].item() - (10 * e[0] + 20 * e[1] + 30 * e[2]) / sum(e)) < 1e-12
    o2 = P.attention(q, k, v, 2)                                                     # window 2: position 2 sees keys 1, 2
    assert abs(o2[2, 0, 0].item() - (20 * e[1] + 30 * e[2]) / (e[1] + e[2])) < 1e-12
    assert torch.equal(o2[:2], o[:2])
    # grouped queries: heads 0,1 read kv head 0; heads 2,3 read kv head 1
    q4 = torch.ones(1, 4, 2, dtype=D)
    kv = torch.tensor([[[1.0, 0.0], [0.0, 1.0]]], dtype=D)
    o4 = P.attention(q4, kv, kv * 5, 0)
    assert o4[0, 0].tolist() == o4[0, 1].tolist() == [5.0, 0.0] and o4[0, 2].tolist() == [0.0, 5.0]


def test_sparsemixer_by_hand():
    # threshold 2*eps = 0.2
    s = torch.tensor([2.0, 1.9, -1.0, 0.5], dtype=D)
    i1, g1, i2, g2 = P.sparsemixer_top2(s, 0.1)
    assert (i1, i2) == (0, 1)
    assert abs(g1.item() - 1 / (1 + math.exp(-0.1))) < 1e-12      # only 1.9 survives the mask beside the winner
    assert abs(g2.item() - 1.0) < 1e-12                            # 0.5 and -1 are masked against 1.9
    # runner-up inside the band of the second selection: (1.9-1.6)/1.9 = 0.158 < 0.2
    s = torch.tensor([2.0, 1.9, 1.6, -4.0], dtype=D)
    _, g1, _, g2 = P.sparsemixer_top2(s, 0.1)
    assert abs(g1.item() - 1 / (1 + math.exp(-0.1) + math.exp(-0.4))) < 1e-12
    assert abs(g2.item() - 1 / (1 + math.exp(-0.3))) < 1e-12
    # negative maximum: the divisor is |s_j|; ties go to the lowest index
    s = torch.tensor([-3.0, -1.0, -1.0, -2.0], dtype=D)
    i1, g1, i2, g2 = P.sparsemixer_top2(s, 0.1)
    assert (i1, i2) == (1, 2)
    assert abs(g1.item() - 0.5) < 1e-12 and abs(g2.item() - 1.0) < 1e-12


def test_expert_and_moe_by_hand():
    x = torch.tensor([[1.0, -1.0]], dtype=D)
    w1 = torch.tensor([[2.0, 0.0]], dtype=D)     # gate pre-activation 2
    w3 = torch.tensor([[0.0, 3.0]], dtype=D)     # up -3
    w2 = torch.tensor([[1.0], [2.0]], dtype=D)
    silu2 = 2 / (1 + math.exp(-2))
    assert torch.allclose(P.expert_mlp(x, w1, w3, w2), torch.tensor([[-3 * silu2, -6 * silu2]], dtype=D))
    # two experts, router picks (0, 1); the second gate is 1 when nothing else is left
    router = torch.tensor([[1.0, 0.0], [0.0, 0.0]], dtype=D)     # logits [1, 0]
    experts = [(w1, w3, w2), (w1 * 0, w3, w2)]
    rec = []
    y = P.moe_feed_forward(x, router, experts, 0.01, record=rec)
    assert [r[:2] for r in rec] == [(0, 1)]
    assert torch.allclose(y, torch.tensor([[-3 * silu2, -6 * silu2]], dtype=D))      # g1 = 1 (other masked), expert 1 gives 0


def test_whole_model_is_causal_and_deterministic(tmp_path):
    import tiny
    folder = tiny.write_tiny(tmp_path / "b", "B", seed=2)
    toks = tiny.random_tokens(90, 384, 1)
    a = P.logits_for(folder, toks)
    b = P.logits_for(folder, toks[:60])
    assert torch.allclose(a[:60], b, atol=1e-12)                  # later tokens do not change earlier logits
    assert a.shape == (90, 384) and torch.isfinite(a).all()
    # the window matters: without it, positions past 48 change
    cfg, w = P.load_model_dir(folder)
    c = P.forward({**cfg, "sliding_window": None}, w, toks)
    assert torch.allclose(c[:48], a[:48], atol=1e-12) and not torch.allclose(c[60:], a[60:], atol=1e-6)


def test_sampler_order_and_filters():
    logits = np.log(np.array([0.5, 0.2, 0.15, 0.1, 0.05], dtype=np.float32))
    s = P.PlainSampler(temperature=1.0, top_k=0, top_p=1.0)
    _, pr = s.probs(logits)
    assert np.allclose(pr, [0.5, 0.2, 0.15, 0.1, 0.05], atol=1e-6)
    _, pr = P.PlainSampler(temperature=1.0, top_k=3, top_p=1.0).probs(logits)
    assert np.allclose(pr, np.array([0.5, 0.2, 0.15, 0, 0]) / 0.85, atol=1e-6)
    _, pr = P.PlainSampler(temperature=1.0, top_k=0, top_p=0.6).probs(logits)       # 0.5 < 0.6 <= 0.7
    assert np.allclose(pr, np.array([0.5, 0.2, 0, 0, 0]) / 0.7, atol=1e-6)
    _, pr = P.PlainSampler(temperature=1.0, top_k=0, top_p=1.0, min_p=0.25).probs(logits)   # floor 0.125
    assert np.allclose(pr, np.array([0.5, 0.2, 0.15, 0, 0]) / 0.85, atol=1e-6)
    tok, _ = P.PlainSampler(temperature=0.0).probs(np.array([1.0, 3.0, 3.0, 2.0], dtype=np.float32))
    assert tok == 1                                                                   # first maximum wins
    # repeat penalty: positive scores are divided, negative multiplied, over the last n generated tokens
    tok, _ = P.PlainSampler(temperature=0.0, repeat_penalty=2.0, repeat_last_n=2).probs(
        np.array([4.0, 3.0, -1.0], dtype=np.float32), context=[0, 1, 2])
    assert tok == 0                        # token 0 is outside the last two; 3.0 -> 1.5, -1 -> -2
    # splitmix64 stream: reproducible, in [0, 1)
    a, b = P.PlainSampler(seed=7), P.PlainSampler(seed=7)
    us = [a.next_f32() for _ in range(5)]
    assert us == [b.next_f32() for _ in range(5)] and all(0 <= u < 1 for u in us) and len(set(us)) == 5
    # draws follow the distribution
    s = P.PlainSampler(temperature=1.0, top_k=0, top_p=1.0, seed=1)
    draws = [s.sample(logits) for _ in range(4000)]
    assert abs(draws.count(0) / 4000 - 0.5) < 0.03 and abs(draws.count(4) / 4000 - 0.05) < 0.02


def test_package_generator_matches_the_plain_one():
    from flint_b200.sampling.params import SplitMix64
    a, b = SplitMix64(43), P.PlainSampler(seed=43)
    assert [a.next_f32() for _ in range(8)] == [float(b.next_f32()) for _ in range(8)]


@pytest.mark.parametrize("which", ["A", "B"])
def test_the_two_plain_implementations_agree(tmp_path, which):
    """The C++ float32 implementation (tests/plain_phimoe.cpp) and the torch float64 one were written
    independently from the same formulas: same logits to float32 accuracy, the same experts everywhere
    (except at a tie within float32 rounding), the same greedy and sampled tokens."""
    import plain_cpp
    import tiny
    folder = tiny.write_tiny(tmp_path / "m", which, seed=13, dtype=torch.float32)
    cfg, w = plain_phimoe.load_model_dir(folder)
    V, L = cfg["vocab_size"], cfg["num_hidden_layers"]
    reqs = [tiny.random_tokens(n, V, 40 + n) for n in ((7, 13, 32) if which == "A" else (5, 40, 70, 100))]
    got = plain_cpp.logits(folder, reqs, L, V)
    for toks, (lg, ex) in zip(reqs, got):
        rec = []
        want = plain_phimoe.forward(cfg, w, toks, rec)
        mine = torch.tensor(lg, dtype=torch.float64).view(len(toks), V)
        err = float((mine - want).abs().max() / want.abs().max())
        assert err < 1e-5, err
        ex = torch.tensor(ex).view(L, len(toks), 2)
        for l in range(L):
            for t in range(len(toks)):
                assert tuple(ex[l, t].tolist()) == rec[l][t][:2] or rec[l][t][4] < 1e-5, (l, t, ex[l, t], rec[l][t])
    # generation: greedy, and temperature 0.8 with the reference's default filters and a fixed seed
    for temperature, k, p in ((0.0, 0, 1.0), (0.8, 20, 0.8)):
        out, _ = plain_cpp.generate(folder, reqs[:2], 6, temperature, k, p, seed=5)
        for i, (prompt, toks) in enumerate(zip(reqs[:2], out)):
            s = plain_phimoe.PlainSampler(temperature, k, p, seed=5 + i + 1)
            seq = list(prompt)
            eos = cfg["eos_token_id"] if isinstance(cfg["eos_token_id"], list) else [cfg["eos_token_id"]]
            for tok in toks:
                want = s.sample(plain_phimoe.forward(cfg, w, seq)[-1].float().numpy())
                assert tok == want
                seq.append(tok)
            assert len(toks) == 6 or s.sample(plain_phimoe.forward(cfg, w, seq)[-1].float().numpy()) in eos
