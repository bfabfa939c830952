"""Phi-MoE (``PhimoeForCausalLM``) as a ``ModelSpec``.

Every layer is a pre-norm block of LayerNorm-with-bias, grouped-query attention with
LongRoPE (optionally windowed, optional q/k/v/o bias), LayerNorm-with-bias, and a
16-expert-style top-2 sparsemixer mixture of SiLU-gated experts; the output head is
untied and may have a bias.  Tensor names are those of the architecture's checkpoints
without the leading ``model.``.  The reference registers its families in one table
keyed by the checkpoint's architecture string
(crates/thuban_architectures/src/loader.rs:39-60); its Phi entry is the dense decoder
(crates/thuban_architectures/src/phi.rs).
"""
from __future__ import annotations

from ..config.phimoe import PhiMoeConfig
from ..config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from ..registry import ARCHITECTURES


@ARCHITECTURES.register("PhimoeForCausalLM")
class PhiMoeArchitecture:
    config_class = PhiMoeConfig

    @staticmethod
    def parse_config(d: dict) -> PhiMoeConfig:
        return PhiMoeConfig.from_dict(d)

    @staticmethod
    def model_spec(cfg: PhiMoeConfig) -> ModelSpec:
        rope = {"rotary_dim": cfg.rotary_dim, "theta": cfg.rope_theta, "max_positions": cfg.max_position_embeddings}
        if cfg.rope_scaling is not None:
            rs = cfg.rope_scaling
            rope.update(short_factor=rs.short_factor, long_factor=rs.long_factor,
                        original_max_positions=rs.original_max_position_embeddings,
                        short_mscale=rs.short_mscale, long_mscale=rs.long_mscale)
        position = PartSpec("rope", rope)
        window = cfg.sliding_window if 0 < cfg.sliding_window < cfg.max_position_embeddings else 0
        norm = PartSpec("layernorm", {"width": cfg.hidden_size, "eps": cfg.layer_norm_eps, "bias": True})
        mixer = PartSpec("attention", {
            "hidden_size": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "window": window,
            "qkv_bias": cfg.attention_bias, "out_bias": cfg.attention_bias, "position": position})
        ffn = PartSpec("sparsemixer_moe", {
            "hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size,
            "num_experts": cfg.num_local_experts, "jitter_eps": cfg.router_jitter_noise, "act": cfg.hidden_act})
        names = {"norm1": "input_layernorm.", "mixer": "self_attn.", "norm2": "post_attention_layernorm.",
                 "ffn": "block_sparse_moe."}
        layers = tuple(LayerSpec("prenorm", {"norm1": norm, "mixer": mixer, "norm2": norm, "ffn": ffn},
                                 f"layers.{i}.", names) for i in range(cfg.num_hidden_layers))
        return ModelSpec(
            architecture=cfg.architecture, vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
            max_positions=cfg.max_position_embeddings, layers=layers,
            order=tuple(LayerCall(i) for i in range(cfg.num_hidden_layers)),
            final_norm=norm, head_bias=cfg.lm_head_bias, tie_word_embeddings=cfg.tie_word_embeddings,
            eos_token_ids=cfg.eos_token_id)
