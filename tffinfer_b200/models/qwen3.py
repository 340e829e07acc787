"""Qwen3 dense as a model description: the counterpart of the reference's creator
(src/core/model/qwen3/QWen3Creator.cpp:15-166), registered under the name that
config.json carries in ``architectures[0]`` the way the reference registers its
creator under the GGUF architecture name (QWen3Creator.cpp:11-12).

Tensor names are the safetensors names of the checkpoint family; the reference's
GGUF names for the same tensors are in src/core/global/ModelGlobalVar.h:206-232
(token_embd, blk.N.attn_norm, attn_q/k/v, attn_q_norm, attn_k_norm, attn_output,
ffn_norm, ffn_gate/up/down, output_norm, output).
"""
from __future__ import annotations

from ..config.model_config import Qwen3Config
from ..parts.description import ModelDescription, LayerSpec, PartSpec, ScheduleEntry
from ..registry import register_architecture

ARCHITECTURE = "Qwen3ForCausalLM"


def describe_qwen3(cfg: Qwen3Config) -> ModelDescription:
    layers = []
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}"
        layers.append(LayerSpec(
            mixer=PartSpec("gqa_attention", dict(
                hidden_size=cfg.hidden_size, num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads,
                head_dim=cfg.head_dim, qk_norm=True, qk_norm_eps=cfg.rms_norm_eps,
                window=cfg.window_of_layer(i)), prefix=f"{p}.self_attn"),
            feed_forward=PartSpec("swiglu", dict(
                hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size), prefix=f"{p}.mlp"),
            mixer_norm=PartSpec("rms_norm", dict(dim=cfg.hidden_size, eps=cfg.rms_norm_eps),
                                prefix=f"{p}.input_layernorm"),
            ffn_norm=PartSpec("rms_norm", dict(dim=cfg.hidden_size, eps=cfg.rms_norm_eps),
                              prefix=f"{p}.post_attention_layernorm"),
            block="pre_norm",
            position="rope"))
    return ModelDescription(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_position=cfg.max_position,
        embed_name="model.embed_tokens.weight",
        lm_head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        final_norm=PartSpec("rms_norm", dict(dim=cfg.hidden_size, eps=cfg.rms_norm_eps), prefix="model.norm"),
        layers=layers,
        schedule=[ScheduleEntry(layer=i) for i in range(cfg.num_layers)],
        positions={"rope": PartSpec("rotary", dict(head_dim=cfg.head_dim, theta=cfg.rope_theta))},
    )


register_architecture(ARCHITECTURE, Qwen3Config.from_json_dict, describe_qwen3, replace=True)
