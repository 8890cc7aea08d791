"""Qwen3 dense decoder (``Qwen3ForCausalLM``) as a model spec.

Tensor names are the checkpoint's own, the ones the reference dereferences as attribute paths
(ampere_kv/runner.py:64-66, 74-75, 118, 165, 170, 174-177, 230, 295, 297).  Every layer is a
pre-norm block of grouped-query attention with per-head QK-norm and rotate-half RoPE, and a
SiLU-gated MLP (runner.py:102-179).  Layers that config.json marks as sliding get a window;
the reference itself refuses such checkpoints (runner.py:39-40).
"""

from __future__ import annotations

from ..config.model_config import Qwen3Config
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .registry import register_architecture


def build_spec(config: Qwen3Config) -> ModelSpec:
    rope = PartSpec("rope", {"theta": config.rope_theta, "rotary_dim": config.head_dim})
    layers = []
    for i in range(config.num_hidden_layers):
        prefix = f"model.layers.{i}"
        mixer = PartSpec("attention", {
            "num_heads": config.num_attention_heads,
            "num_kv_heads": config.num_key_value_heads,
            "head_dim": config.head_dim,
            "qk_norm": True,
            "qk_norm_eps": config.rms_norm_eps,
            "bias": config.attention_bias,
            "window": config.window_of_layer(i),
            "scale": None,
            "position_encoding": rope,
        }, f"{prefix}.self_attn")
        ff = PartSpec("gated_mlp", {"intermediate_size": config.intermediate_size,
                                    "activation": config.hidden_act}, f"{prefix}.mlp")
        layers.append(LayerSpec(
            block="prenorm", mixer=mixer, feed_forward=ff,
            mixer_norm=PartSpec("rmsnorm", {"eps": config.rms_norm_eps}, f"{prefix}.input_layernorm"),
            feed_forward_norm=PartSpec("rmsnorm", {"eps": config.rms_norm_eps},
                                       f"{prefix}.post_attention_layernorm")))
    return ModelSpec(
        hidden_size=config.hidden_size,
        vocab_size=config.vocab_size,
        embedding=PartSpec("token_embedding", {"vocab_size": config.vocab_size}, "model.embed_tokens"),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(config.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", {"eps": config.rms_norm_eps}, "model.norm"),
        head=PartSpec("linear_head", {"vocab_size": config.vocab_size, "tied": config.tie_word_embeddings},
                      "lm_head"),
        max_position=config.max_position_embeddings,
        eos_token_ids=config.eos_token_id,
    )


register_architecture("Qwen3ForCausalLM", Qwen3Config, build_spec)
