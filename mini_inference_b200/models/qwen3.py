"""Qwen3 dense: configuration -> ModelSpec.

Layer make-up as the reference runs it (engine/core/model_runner.py:112-196): pre-norm
residual block; grouped-query attention with one RMSNorm weight vector per q and per k
shared by all heads, applied before rotate-half RoPE (:148-152); SwiGLU feed-forward
(:124-131); final RMSNorm and a head that is the embedding matrix when tied (:133-135).
Tensor names are the checkpoint's own (model.layers.{i}.self_attn.q_proj.weight, ...).
"""
from __future__ import annotations

from ..config.model_config import Qwen3Config
from ..config.registry import register_architecture
from ..config.spec import ExecStep, LayerSpec, ModelSpec, PartSpec


def build_spec(cfg: Qwen3Config) -> ModelSpec:
    norm = PartSpec.of("rmsnorm", size=cfg.hidden_size, eps=cfg.rms_norm_eps)
    position = PartSpec.of("rotary", head_dim=cfg.head_dim, theta=cfg.rope_theta)
    feed_forward = PartSpec.of("swiglu", hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size)
    layers = []
    for i in range(cfg.num_hidden_layers):
        mixer = PartSpec.of(
            "gqa_attention", hidden_size=cfg.hidden_size, num_heads=cfg.num_attention_heads,
            num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
            scale=cfg.head_dim ** -0.5, qk_norm=True, qk_norm_eps=cfg.rms_norm_eps,
            window=cfg.layer_windows[i])
        p = f"model.layers.{i}."
        names = {
            "norm1.weight": p + "input_layernorm.weight",
            "norm2.weight": p + "post_attention_layernorm.weight",
            "mixer.q_proj": p + "self_attn.q_proj.weight", "mixer.k_proj": p + "self_attn.k_proj.weight",
            "mixer.v_proj": p + "self_attn.v_proj.weight", "mixer.o_proj": p + "self_attn.o_proj.weight",
            "mixer.q_norm": p + "self_attn.q_norm.weight", "mixer.k_norm": p + "self_attn.k_norm.weight",
            "feed_forward.gate_proj": p + "mlp.gate_proj.weight",
            "feed_forward.up_proj": p + "mlp.up_proj.weight",
            "feed_forward.down_proj": p + "mlp.down_proj.weight",
        }
        layers.append(LayerSpec.of("prenorm", names, mixer=mixer, feed_forward=feed_forward, norm1=norm, norm2=norm,
                                   position=position))
    return ModelSpec(
        hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size, layers=tuple(layers),
        order=tuple(ExecStep(i) for i in range(cfg.num_hidden_layers)),
        final_norm=norm, embedding_name="model.embed_tokens.weight", final_norm_name="model.norm.weight",
        lm_head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        max_position=cfg.max_position_embeddings, eos_token_ids=cfg.eos_token_ids)


register_architecture("Qwen3ForCausalLM", "Qwen3 dense (GQA, per-head q/k norm)", Qwen3Config, build_spec)
