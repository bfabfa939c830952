"""Configuration reading and the architecture registry (no GPU)."""
import json

import pytest

import flint_b200  # noqa: F401
from flint_b200.config.phimoe import PhiMoeConfig
from flint_b200.engine.model import architecture_of
from flint_b200.errors import ConfigError
from flint_b200.registry import ARCHITECTURES, MIXERS
from tiny import TINY_A, TINY_B


def test_reads_every_key_of_both_tiny_configs():
    a, b = PhiMoeConfig.from_dict(TINY_A), PhiMoeConfig.from_dict(TINY_B)
    assert (a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (64, 4, 2, 16)
    assert (b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (96, 3, 1, 32)
    assert a.rope_scaling is None and a.sliding_window == 0 and a.attention_bias and a.lm_head_bias
    assert b.sliding_window == 48 and not b.attention_bias and not b.lm_head_bias
    assert a.layer_norm_eps == 1e-5 and b.layer_norm_eps == 1e-6
    assert a.router_jitter_noise == 0.01 and b.router_jitter_noise == 0.05
    assert a.eos_token_id == (2,) and b.eos_token_id == (1, 2)
    rs = b.rope_scaling
    assert rs.original_max_position_embeddings == 64 and len(rs.short_factor) == 16
    # scale from the ratio of the two context lengths: sqrt(1 + ln(512/64)/ln(64)) = sqrt(1.5)
    assert abs(rs.long_mscale - 1.5 ** 0.5) < 1e-12 and rs.short_mscale == rs.long_mscale


def test_defaults_and_aliases():
    d = dict(TINY_A)
    for k in ("head_dim", "rms_norm_eps", "router_jitter_noise", "sliding_window", "attention_bias"):
        d.pop(k)
    d["layer_norm_epsilon"] = 3e-5
    d["jitter_eps"] = 0.2
    c = PhiMoeConfig.from_dict(d)
    assert c.head_dim == 16 and c.layer_norm_eps == 3e-5 and c.router_jitter_noise == 0.2
    assert c.sliding_window == 0 and c.attention_bias is False and c.tie_word_embeddings is False
    d2 = dict(TINY_B)
    d2["rope_scaling"] = dict(d2["rope_scaling"], short_mscale=1.1, long_mscale=1.3,
                              original_max_position_embeddings=32)
    c2 = PhiMoeConfig.from_dict(d2)
    assert (c2.rope_scaling.short_mscale, c2.rope_scaling.long_mscale) == (1.1, 1.3)
    assert c2.rope_scaling.original_max_position_embeddings == 32


def test_round_trip_through_json(tmp_path):
    for cfg in (TINY_A, TINY_B):
        c = PhiMoeConfig.from_dict(cfg)
        p = tmp_path / "config.json"
        p.write_text(json.dumps(c.to_dict()))
        assert PhiMoeConfig.from_json(p) == c


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "vocab_size", "rope_theta",
                                 "num_local_experts", "intermediate_size", "max_position_embeddings"])
def test_missing_key_is_named(key):
    d = dict(TINY_A)
    d.pop(key)
    with pytest.raises(ConfigError, match=key):
        PhiMoeConfig.from_dict(d)


@pytest.mark.parametrize("patch,match", [
    ({"hidden_size": "64"}, "hidden_size"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"hidden_act": "relu"}, "hidden_act"),
    ({"num_experts_per_tok": 3}, "num_experts_per_tok"),
    ({"partial_rotary_factor": 0.2}, "partial_rotary_factor"),
    ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"rope_scaling": {"type": "longrope", "short_factor": [1.0] * 3, "long_factor": [1.0] * 8}}, "short_factor"),
    ({"attention_bias": 1}, "attention_bias"),
    ({"eos_token_id": "x"}, "eos_token_id"),
])
def test_bad_values_are_refused(patch, match):
    with pytest.raises(ConfigError, match=match):
        PhiMoeConfig.from_dict({**TINY_A, **patch})


def test_head_dim_needs_divisibility():
    d = dict(TINY_A, hidden_size=66)
    d.pop("head_dim")
    with pytest.raises(ConfigError, match="divisible"):
        PhiMoeConfig.from_dict(d)


def test_registry_maps_name_to_model_and_lists_known_names():
    arch = architecture_of(TINY_A)
    assert arch is ARCHITECTURES.get("PhimoeForCausalLM")
    with pytest.raises(ConfigError, match="PhimoeForCausalLM"):
        architecture_of({"architectures": ["NoSuchModel"]})
    with pytest.raises(ConfigError, match="architectures"):
        architecture_of({})
    with pytest.raises(ConfigError, match="attention"):
        MIXERS.get("no_such_mixer")


def test_model_spec_has_no_size_of_its_own():
    for cfg in (TINY_A, TINY_B):
        arch = architecture_of(cfg)
        c = arch.parse_config(cfg)
        spec = arch.model_spec(c)
        assert len(spec.layers) == c.num_hidden_layers == len(spec.order)
        m = spec.layers[0].parts["mixer"].params
        assert (m["num_heads"], m["num_kv_heads"], m["head_dim"]) == (c.num_attention_heads, c.num_key_value_heads, c.head_dim)
        f = spec.layers[0].parts["ffn"].params
        assert (f["num_experts"], f["intermediate_size"], f["jitter_eps"]) == (c.num_local_experts, c.intermediate_size, c.router_jitter_noise)
        assert spec.layers[0].parts["norm1"].params["eps"] == c.layer_norm_eps
        assert m["window"] == c.sliding_window
