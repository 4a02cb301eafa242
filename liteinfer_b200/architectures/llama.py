"""The dense grouped-query Llama decoder as a `ModelSpec`.

liteinfer/models/llama.py: token embedding (:204), per layer a pre-norm
residual block of grouped-query attention with rotary embeddings and a SwiGLU
MLP (:166-192), a final RMSNorm (:208,228) and a linear head, tied to the
embedding when `tie_word_embeddings` (:245-247).  Tensor names are the
checkpoint's own (HF names, liteinfer/models/loader.py:49-72).
"""

from __future__ import annotations

from liteinfer_b200.config.model_config import LlamaConfig
from liteinfer_b200.config.registry import register_architecture
from liteinfer_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def llama_spec(config: LlamaConfig) -> ModelSpec:
    scaling = config.rope_scaling
    position = PartSpec("rotary", {
        "head_dim": config.head_dim, "theta": config.rope_theta, "rope_type": scaling.rope_type,
        "factor": scaling.factor, "low_freq_factor": scaling.low_freq_factor,
        "high_freq_factor": scaling.high_freq_factor,
        "original_max_position_embeddings": scaling.original_max_position_embeddings,
    })
    norm = PartSpec("rmsnorm", {"size": config.hidden_size, "eps": config.rms_norm_eps})
    mixer = PartSpec("attention", {
        "hidden_size": config.hidden_size, "heads": config.num_attention_heads,
        "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim, "position": position,
        "bias": config.attention_bias,
    })
    feed_forward = PartSpec("gated_mlp", {
        "hidden_size": config.hidden_size, "intermediate_size": config.intermediate_size,
        "activation": config.hidden_act, "bias": config.mlp_bias,
    })
    layers = tuple(
        LayerSpec(
            block="prenorm_residual",
            parts={"mixer_norm": norm, "mixer": mixer, "feed_forward_norm": norm, "feed_forward": feed_forward},
            prefixes={
                "mixer_norm": f"model.layers.{i}.input_layernorm.",
                "mixer": f"model.layers.{i}.self_attn.",
                "feed_forward_norm": f"model.layers.{i}.post_attention_layernorm.",
                "feed_forward": f"model.layers.{i}.mlp.",
            },
        )
        for i in range(config.num_hidden_layers)
    )
    sizes = {"vocab_size": config.vocab_size, "hidden_size": config.hidden_size}
    return ModelSpec(
        vocab_size=config.vocab_size,
        hidden_size=config.hidden_size,
        embedding=PartSpec("token_embedding", sizes),
        embedding_prefix="model.embed_tokens.",
        layers=layers,
        schedule=tuple(ScheduleEntry(i) for i in range(config.num_hidden_layers)),
        final_norm=norm,
        final_norm_prefix="model.norm.",
        head=PartSpec("linear", sizes),
        head_prefix="lm_head.",
        tied={"lm_head.weight": "model.embed_tokens.weight"} if config.tie_word_embeddings else {},
    )


register_architecture("LlamaForCausalLM", LlamaConfig, llama_spec, replace=True)
