"""Typed configuration of Phi-MoE (``PhimoeForCausalLM``), read from the keys of its
own config.json.

The dense part of the key set and the defaults follow the reference's Phi parser
(crates/thuban_architectures/src/phi.rs:13-80 and
crates/thuban_architectures/src/transformer/config.rs:70-138); the keys for the
experts, the sliding window, the LongRoPE magnitude scale and the head bias are the
architecture's own.
"""
from __future__ import annotations

import json
import math
from dataclasses import asdict, dataclass
from pathlib import Path

from ..errors import ConfigError
from . import fields as F


@dataclass(frozen=True)
class LongRopeScaling:
    short_factor: tuple
    long_factor: tuple
    original_max_position_embeddings: int
    short_mscale: float
    long_mscale: float


@dataclass(frozen=True)
class PhiMoeConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rope_theta: float
    partial_rotary_factor: float
    rope_scaling: LongRopeScaling | None
    sliding_window: int            # 0 = none
    layer_norm_eps: float
    hidden_act: str
    attention_bias: bool
    lm_head_bias: bool
    tie_word_embeddings: bool
    num_local_experts: int
    num_experts_per_tok: int
    router_jitter_noise: float
    eos_token_id: tuple
    architecture: str = "PhimoeForCausalLM"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: dict) -> "PhiMoeConfig":
        hidden = F.get_int(d, "hidden_size", minimum=1)
        nq = F.get_int(d, "num_attention_heads", minimum=1)
        if "head_dim" in d and d["head_dim"] is not None:
            hd = F.get_int(d, "head_dim", minimum=1)
        else:
            if hidden % nq:
                raise ConfigError("hidden_size not divisible by num_attention_heads and no head_dim given")
            hd = hidden // nq
        nkv = F.get_int(d, "num_key_value_heads", default=nq, minimum=1)
        if nq % nkv:
            raise ConfigError(f"num_attention_heads ({nq}) must be a multiple of num_key_value_heads ({nkv})")
        max_pos = F.get_int(d, "max_position_embeddings", minimum=1)
        partial = F.get_float(d, "partial_rotary_factor", default=1.0)
        rot = int(hd * partial)
        if rot <= 0 or rot > hd or rot % 2:
            raise ConfigError(f"invalid partial_rotary_factor {partial} for head_dim {hd}")
        scaling = None
        rs = d.get("rope_scaling")
        if rs is not None:
            if not isinstance(rs, dict):
                raise ConfigError("config field 'rope_scaling' must be an object")
            kind = rs.get("type", rs.get("rope_type", "longrope"))
            if kind != "longrope":
                raise ConfigError(f"unsupported rope_scaling type {kind!r} (supported: 'longrope')")
            if "original_max_position_embeddings" in rs:
                orig = F.get_int(rs, "original_max_position_embeddings", minimum=2)
            else:
                orig = F.get_int(d, "original_max_position_embeddings", default=4096, minimum=2)
            default_m = (math.sqrt(1.0 + math.log(max_pos / orig) / math.log(orig))
                         if max_pos > orig else 1.0)
            scaling = LongRopeScaling(
                short_factor=F.get_float_list(rs, "short_factor", length=rot // 2),
                long_factor=F.get_float_list(rs, "long_factor", length=rot // 2),
                original_max_position_embeddings=orig,
                short_mscale=F.get_float(rs, "short_mscale", default=default_m),
                long_mscale=F.get_float(rs, "long_mscale", default=default_m),
            )
        act = F.get_str(d, "hidden_act", default="silu")
        if act not in ("silu", "gelu_pytorch_tanh"):
            raise ConfigError(f"unsupported hidden_act {act!r} (supported: silu, gelu_pytorch_tanh)")
        k = F.get_int(d, "num_experts_per_tok", default=2)
        if k != 2:
            raise ConfigError(f"num_experts_per_tok must be 2 (sparsemixer routing), got {k}")
        E = F.get_int(d, "num_local_experts", minimum=2)
        arch = d.get("architectures") or ["PhimoeForCausalLM"]
        return cls(
            vocab_size=F.get_int(d, "vocab_size", minimum=1),
            hidden_size=hidden,
            intermediate_size=F.get_int(d, "intermediate_size", minimum=1),
            num_hidden_layers=F.get_int(d, "num_hidden_layers", minimum=1),
            num_attention_heads=nq,
            num_key_value_heads=nkv,
            head_dim=hd,
            max_position_embeddings=max_pos,
            rope_theta=F.get_float(d, "rope_theta"),
            partial_rotary_factor=partial,
            rope_scaling=scaling,
            sliding_window=F.get_int(d, "sliding_window", default=0, minimum=0),
            layer_norm_eps=F.get_float(d, "rms_norm_eps", default=1e-5,
                                       aliases=("layer_norm_eps", "layer_norm_epsilon")),
            hidden_act=act,
            attention_bias=F.get_bool(d, "attention_bias", default=False),
            lm_head_bias=F.get_bool(d, "lm_head_bias", default=False),
            tie_word_embeddings=F.get_bool(d, "tie_word_embeddings", default=False),
            num_local_experts=E,
            num_experts_per_tok=k,
            router_jitter_noise=F.get_float(d, "router_jitter_noise", default=0.01, aliases=("jitter_eps",)),
            eos_token_id=F.get_int_list(d, "eos_token_id"),
            architecture=arch[0],
        )

    @classmethod
    def from_json(cls, path) -> "PhiMoeConfig":
        return cls.from_dict(json.loads(Path(path).read_text()))

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        d = asdict(self)
        d.pop("architecture")
        d["architectures"] = [self.architecture]
        d["model_type"] = "phimoe"
        d["rms_norm_eps"] = d.pop("layer_norm_eps")
        d["eos_token_id"] = list(self.eos_token_id) or None
        if self.sliding_window == 0:
            d["sliding_window"] = None
        if self.rope_scaling is not None:
            rs = asdict(self.rope_scaling)
            rs["type"] = "longrope"
            rs["short_factor"] = list(rs["short_factor"])
            rs["long_factor"] = list(rs["long_factor"])
            d["rope_scaling"] = rs
            d["original_max_position_embeddings"] = self.rope_scaling.original_max_position_embeddings
        return d

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)
