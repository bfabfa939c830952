"""The engine at the layer sizes it is measured at (Phi-mini-MoE: width 4096, 32 query heads on 8 KV heads of
128, 16 experts of 960, vocabulary 32064, LongRoPE 4096 -> 131072, biases on), 2 of the 32 layers, against the
plain implementation, in 32-bit and in bfloat16, under every way of cutting the work.

The tiny configurations cannot reach what runs here: K loops of 64 blocks through the rings of the tensor-core
products, K ranges split over blocks, the expert products cut stream-K fashion, the vocabulary's ragged last
tile, prefill tiles of 256 rows per expert, 2,048-token portions beside decoded tokens, positions past the
original context (the long factors), and decode batches of eight through the captured graph."""
import random

import pytest
import torch

import plain_phimoe
import traces
from engine_checks import compare, plain_all, replay
from flint_b200.engine.loading import write_random_model

pytestmark = pytest.mark.gpu


def _factors(n, seed):
    r = random.Random(seed)
    return [round(r.uniform(1.0, 4.0), 4) for _ in range(n)]


MINI_2_OF_32 = {
    "architectures": ["PhimoeForCausalLM"], "model_type": "phimoe",
    "vocab_size": 32064, "hidden_size": 4096, "intermediate_size": 960, "num_hidden_layers": 2,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "max_position_embeddings": 131072, "original_max_position_embeddings": 4096, "rope_theta": 10000.0,
    "rope_scaling": {"type": "longrope", "short_factor": _factors(64, 1), "long_factor": _factors(64, 2)},
    "sliding_window": 131072, "rms_norm_eps": 1e-5, "hidden_act": "silu",
    "attention_bias": True, "lm_head_bias": True, "tie_word_embeddings": False,
    "num_local_experts": 16, "num_experts_per_tok": 2, "router_jitter_noise": 0.01, "eos_token_id": 2,
}
LENGTHS = (300, 700, 2100, 4200)                 # the last one crosses the original context of 4096
SHORT = (40, 75, 130, 61, 222, 97, 160, 33)      # eight more, decoded together


# With random weights of these sizes a router logit carries about 0.6 % of bfloat16 noise (the attention's
# probabilities, keys and values are all rounded), and the gaps between the sixteen logits of a row are dense
# enough near zero that several per cent of the decisions sit inside that noise.  Every differing decision
# still has to be proven a near-tie from the engine's own router logits (engine_checks.plain_following); this
# only bounds how many there may be.
DIFFERING = {"float32": 0.0005, "bfloat16": 0.10}


def kept_positions(n):
    """The positions of a request of n tokens whose logits are compared: the first ones, every 61st, the
    ones around the original context's end, and the last 36 (all of the decoded tail)."""
    keep = set(range(min(n, 3))) | set(range(0, n, 61)) | set(range(max(n - 36, 0), n))
    keep |= {p for p in range(4090, 4102) if p < n}
    return keep


@pytest.fixture(scope="module")
def big(tmp_path_factory):
    # stored in bfloat16: the bfloat16 engine keeps the tensors, the 32-bit engine and the plain implementation
    # widen the same values
    folder = write_random_model(tmp_path_factory.mktemp("mini2"), MINI_2_OF_32, seed=21, dtype=torch.bfloat16)
    reqs = traces.make_requests(MINI_2_OF_32["vocab_size"], LENGTHS + SHORT, seed=17)
    keep = {rid: kept_positions(len(t)) for rid, t in reqs.items()}
    loaded = plain_phimoe.load_model_dir(folder)
    plain = plain_all(folder, reqs, keep, loaded)
    return folder, reqs, keep, plain, loaded


def _long(reqs):
    return {rid: reqs[rid] for rid in list(reqs)[:len(LENGTHS)]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
def test_real_sizes_match_plain_under_every_cut(big, cut, dtype):
    folder, reqs, keep, plain, loaded = big
    reqs = _long(reqs)
    steps = {"whole": lambda r: traces.whole(r, keep=keep),
             "tail": lambda r: traces.tail_decoded(r, keep=keep),
             "portions": lambda r: traces.portions(r, sizes=(2048, 2, 7, 333, 3, 64, 2, 13, 1000, 5, 129, 2), keep=keep),
             # up to four live: portions of 2,048 and of a few tokens beside the decoded tokens of the others
             "mixed": lambda r: traces.mixed(r, seed=4, decode_tail=24, sizes=(2, 3, 16, 33, 257, 2048, 2048), keep=keep),
             }[cut](reqs)
    if cut == "mixed":
        assert any(len(s["entries"]) > 1 and max(len(e["tokens"]) for e in s["entries"]) == 2048
                   and min(len(e["tokens"]) for e in s["entries"]) == 1 for s in steps), \
            "the trace has no 2,048-token portion beside a decoded token"
    out, rp = replay(folder, dtype, steps, 64)
    compare(out, steps, plain, dtype, rp.routing, reqs, folder, keep, loaded, rp.router_logits, DIFFERING[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_sizes_eight_requests_decoded_together(big, dtype):
    """Eight live requests: their prompts in one step, then one token each per step through the captured graph."""
    folder, reqs, keep, plain, loaded = big
    reqs = {rid: reqs[rid] for rid in list(reqs)[len(LENGTHS):]}
    tail = 24
    steps = [{"step": 0, "entries": [{"id": rid, "tokens": t[:-tail], "want": traces._wanted(rid, 0, [len(t) - tail - 1], keep)}
                                     for rid, t in reqs.items()], "end": []}]
    for j in range(tail):
        steps.append({"step": len(steps), "end": list(reqs) if j == tail - 1 else [],
                      "entries": [{"id": rid, "tokens": [t[len(t) - tail + j]], "want": [0]} for rid, t in reqs.items()]})
    out, rp = replay(folder, dtype, steps, 64, max_requests=8)
    assert any(k[0] == 8 for k in rp.model._graphs), "the batch of eight did not go through the captured graph"
    compare(out, steps, plain, dtype, rp.routing, reqs, folder, keep, loaded, rp.router_logits, DIFFERING[dtype])


@pytest.fixture(scope="module")
def windowed(tmp_path_factory):
    """The same layer sizes with a sliding window of 1,000 positions (not a multiple of the page or of a key tile)."""
    cfg = dict(MINI_2_OF_32, sliding_window=1000)
    folder = write_random_model(tmp_path_factory.mktemp("mini2w"), cfg, seed=22, dtype=torch.bfloat16)
    reqs = traces.make_requests(cfg["vocab_size"], (2100, 1300), seed=19)
    keep = {rid: kept_positions(len(t)) | set(range(990, 1012)) for rid, t in reqs.items()}
    loaded = plain_phimoe.load_model_dir(folder)
    return folder, reqs, keep, plain_all(folder, reqs, keep, loaded), loaded


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", ["tail", "mixed"])
def test_real_sizes_with_a_window(windowed, cut, dtype):
    """Prompts twice the window: the tensor-core attention's tiles at the window's edge, decoded tokens whose first
    visible key lies inside a page, and pages behind the window given back and used again."""
    folder, reqs, keep, plain, loaded = windowed
    steps = {"tail": lambda r: traces.tail_decoded(r, keep=keep),
             "mixed": lambda r: traces.mixed(r, seed=6, decode_tail=24, sizes=(2, 16, 33, 257, 700), keep=keep)}[cut](reqs)
    out, rp = replay(folder, dtype, steps, 64)
    compare(out, steps, plain, dtype, rp.routing, reqs, folder, keep, loaded, rp.router_logits, DIFFERING[dtype])
    if cut == "mixed":
        assert max(rp.model.cache.groups[0].pages.pool.served) >= 2, "no page behind the window was used again"
