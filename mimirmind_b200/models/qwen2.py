"""The Qwen2.5 dense decoder, laid out from parts.

What the reference's backend for this architecture does per layer
(src/runtime/arch/Qwen2Backend.cpp:132-466): RMSNorm → q/k/v projections with bias →
split-half RoPE on q and k → cache write → causal GQA attention → output projection →
residual → RMSNorm → SwiGLU → residual; then a final RMSNorm and the output head, tied to
the embedding table when the checkpoint has no head tensor
(src/runtime/InferenceEngine.cpp:1374-1377).  Tensor names are the HF names of the
checkpoint, by the pattern of the reference's HF name table
(src/core/modelopt/Qwen3_5MoeGgufMap.cpp:13-22, 61-65, 81-85).

This module only *describes* the model; it holds no arithmetic.
"""
from __future__ import annotations

from ..config.model_config import Qwen2Config, parse_qwen2_config
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..registry import register_architecture

ARCHITECTURE = "Qwen2ForCausalLM"


def build_spec(cfg: Qwen2Config) -> ModelSpec:
    d = cfg.hidden_size
    layers = []
    for i in range(cfg.num_hidden_layers):
        position = PartSpec("rotary_half", {"theta": cfg.rope_theta, "rotary_dim": cfg.head_dim})
        mixer = PartSpec("gqa_attention", {
            "hidden": d,
            "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim,
            "window": cfg.layer_windows[i],
            "scale": None,
            "qkv_bias": True,
            "position": position,
            "q": "self_attn.q_proj", "k": "self_attn.k_proj", "v": "self_attn.v_proj", "o": "self_attn.o_proj",
        })
        ffn = PartSpec("swiglu", {
            "hidden": d, "intermediate": cfg.intermediate_size,
            "gate": "mlp.gate_proj.weight", "up": "mlp.up_proj.weight", "down": "mlp.down_proj.weight",
        })
        layers.append(LayerSpec(
            prefix=f"model.layers.{i}.",
            block=PartSpec("pre_norm", {}),
            mixer=mixer,
            feed_forward=ffn,
            mixer_norm=PartSpec("rmsnorm", {"width": d, "eps": cfg.rms_norm_eps, "weight": "input_layernorm.weight"}),
            ffn_norm=PartSpec("rmsnorm", {"width": d, "eps": cfg.rms_norm_eps, "weight": "post_attention_layernorm.weight"}),
        ))
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=d,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab_size, "width": d, "scale": 1.0,
                                               "weight": "model.embed_tokens.weight"}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", {"width": d, "eps": cfg.rms_norm_eps, "weight": "model.norm.weight"}),
        head=PartSpec("lm_head", {"vocab": cfg.vocab_size, "width": d, "weight": "lm_head.weight",
                                  "tied_to": "model.embed_tokens.weight" if cfg.tie_word_embeddings else None}),
        eos_token_ids=cfg.eos_token_ids,
    )


register_architecture(ARCHITECTURE, parse_qwen2_config, build_spec)
