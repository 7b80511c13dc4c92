"""Qwen3 dense decoder as a plan of parts (reference: models/qwen3.py:12-116).

Every layer: RMSNorm -> grouped-query attention with per-head q/k RMSNorm and rotary
embedding -> RMSNorm -> SwiGLU, with one rotary table shared by all layers
(models/qwen3.py:81,83), a final RMSNorm and a tied or untied head.  All numbers come
from the configuration.
"""
from __future__ import annotations

from ..config.model_config import Qwen3Config
from ..config.registry import Architecture, register_architecture
from ..parts import BlockSpec, LayerCall, ModelPlan, PartSpec, SharedRef


def qwen3_plan(cfg: Qwen3Config) -> ModelPlan:
    norm = PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    blocks = []
    for i in range(cfg.num_hidden_layers):
        mixer = PartSpec("gqa_attention", {
            "hidden_size": cfg.hidden_size,
            "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim,
            "qk_norm_eps": cfg.rms_norm_eps,
            "position_encoding": SharedRef("rope"),
            "window": cfg.window_of_layer(i),
        })
        ffn = PartSpec("swiglu", {"hidden_size": cfg.hidden_size,
                                  "intermediate_size": cfg.intermediate_size})
        blocks.append(BlockSpec(mixer=mixer, feed_forward=ffn, norm=norm))
    return ModelPlan(
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        blocks=blocks,
        schedule=[LayerCall(i, i, True) for i in range(cfg.num_hidden_layers)],
        final_norm=norm,
        tie_word_embeddings=cfg.tie_word_embeddings,
        max_position=cfg.max_position_embeddings,
        shared={"rope": PartSpec("rope", {"rotary_dim": cfg.head_dim,
                                          "max_position": cfg.max_position_embeddings,
                                          "theta": cfg.rope_theta})},
    )


register_architecture(Architecture("Qwen3ForCausalLM", Qwen3Config.from_dict, qwen3_plan), replace=True)
