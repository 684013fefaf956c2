"""Qwen3 (dense): config.json -> plan.

One decoder layer is add+RMSNorm, grouped-query attention with per-head q/k RMSNorm and
rotate-half position encoding, add+RMSNorm, SwiGLU (vllm-oxide, crates/vllm-oxide/src/models/qwen3.rs:60-305);
the tensors keep their checkpoint names (model.layers.N.self_attn.q_proj.weight, ...).  As in
the reference, q_norm/k_norm exist exactly when there is no q/k/v bias (qwen3.rs:124-139).
Layers from `max_window_layers` on use a sliding window when `use_sliding_window` is set.
"""
from __future__ import annotations

from ..config.model_config import Qwen3Config
from ..parts.base import PartSpec
from .plan import ExecStep, ModelPlan


def qwen3_plan(cfg: Qwen3Config) -> ModelPlan:
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        mixer = PartSpec("attention", dict(
            hidden_size=cfg.hidden_size, num_heads=cfg.num_attention_heads, num_kv_heads=cfg.num_key_value_heads,
            head_dim=cfg.head_dim, eps=cfg.rms_norm_eps, qkv_bias=cfg.attention_bias, qk_norm=not cfg.attention_bias,
            window=cfg.layer_window(i), position="rope", prefix=p + "self_attn."))
        ffn = PartSpec("swiglu", dict(hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
                                      prefix=p + "mlp."))
        norm1 = PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps,
                                         weight_name=p + "input_layernorm.weight"))
        norm2 = PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps,
                                         weight_name=p + "post_attention_layernorm.weight"))
        layers.append(PartSpec("pre_norm", dict(mixer=mixer, feed_forward=ffn, input_norm=norm1,
                                                post_mixer_norm=norm2)))
    return ModelPlan(
        architecture=cfg.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_position=cfg.max_position_embeddings,
        embedding_name="model.embed_tokens.weight",
        lm_head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        final_norm=PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps, weight_name="model.norm.weight")),
        positions={"rope": PartSpec("rope", dict(head_dim=cfg.head_dim, max_position=cfg.max_position_embeddings,
                                                 theta=cfg.rope_theta))},
        layers=layers,
        order=[ExecStep(i, i, True) for i in range(cfg.num_hidden_layers)],
        eos_token_id=cfg.eos_token_id,
        default_dtype=cfg.torch_dtype,
    )
