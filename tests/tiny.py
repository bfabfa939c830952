"""Two tiny Phi-MoE configurations that differ in every size and option, and helpers
that write them as model folders with seeded random weights."""
from __future__ import annotations

import random

import torch

# A: 2 layers, width 64, 4 query heads on 2 KV heads of size 16, 4 experts, no rope scaling,
#    no window, biases on, eps 1e-5.
TINY_A = {
    "architectures": ["PhimoeForCausalLM"], "model_type": "phimoe",
    "vocab_size": 512, "hidden_size": 64, "intermediate_size": 96, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "max_position_embeddings": 256, "rope_theta": 10000.0, "rope_scaling": None,
    "sliding_window": None, "rms_norm_eps": 1e-5, "hidden_act": "silu",
    "attention_bias": True, "lm_head_bias": True, "tie_word_embeddings": False,
    "num_local_experts": 4, "num_experts_per_tok": 2, "router_jitter_noise": 0.01,
    "eos_token_id": 2,
}


def _factors(n, seed):
    r = random.Random(seed)
    return [round(r.uniform(1.0, 4.0), 6) for _ in range(n)]


# B: 3 layers, width 96, 3 query heads on 1 KV head of size 32, 6 experts, LongRoPE crossing its
#    original context (64 -> 512) with the scale derived from the ratio, window 48, no biases, eps 1e-6.
TINY_B = {
    "architectures": ["PhimoeForCausalLM"], "model_type": "phimoe",
    "vocab_size": 384, "hidden_size": 96, "intermediate_size": 80, "num_hidden_layers": 3,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32,
    "max_position_embeddings": 512, "original_max_position_embeddings": 64, "rope_theta": 500000.0,
    "rope_scaling": {"type": "longrope", "short_factor": _factors(16, 1), "long_factor": _factors(16, 2)},
    "sliding_window": 48, "rms_norm_eps": 1e-6, "hidden_act": "silu",
    "attention_bias": False, "lm_head_bias": False, "tie_word_embeddings": False,
    "num_local_experts": 6, "num_experts_per_tok": 2, "router_jitter_noise": 0.05,
    "eos_token_id": [1, 2],
}

CONFIGS = {"A": TINY_A, "B": TINY_B}


def write_tiny(tmp_dir, which="A", seed=0, dtype=torch.float32, overrides=None):
    """Write config.json + model.safetensors for a tiny configuration; returns the folder."""
    from flint_b200.engine.loading import write_random_model
    cfg = dict(CONFIGS[which])
    cfg.update(overrides or {})
    return write_random_model(tmp_dir, cfg, seed=seed, dtype=dtype)


def random_tokens(n, vocab, seed):
    r = random.Random(seed)
    return [r.randrange(vocab) for _ in range(n)]
