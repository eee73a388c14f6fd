"""Gemma-2 as data: the function from a `Gemma2Config` to a `ModelPlan`.

Layer by layer (order as the reference runs it, src/forward.rs:289-415):
input norm -> attention (rotary q/k, scale, soft-cap, causal or windowed) ->
post-attention norm -> residual; pre-feed-forward norm -> GeGLU -> post-feed-
forward norm -> residual.  All norms are RMSNorm with the weight applied as
(1 + w) (src/hf.rs:101-107).  The embedding is scaled by sqrt(hidden)
(src/model.rs:899), the head reuses the embedding table unless the checkpoint
has `lm_head.weight` (src/model.rs:879-883), and the logits are soft-capped
(src/forward.rs:431-435).  Tensor names are the checkpoint's own
(src/hf.rs:216-364).
"""
from __future__ import annotations

import math

from ..config.base import LayerCall, LayerSpec, ModelPlan, PartSpec
from ..config.gemma2 import Gemma2Config
from ..registry import register_architecture


def gemma2_plan(cfg: Gemma2Config) -> ModelPlan:
    width = cfg.hidden_size

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"width": width, "eps": cfg.rms_norm_eps, "add_one": True},
                        {"weight": name})

    layers = []
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        position = PartSpec("rotary", {"theta": cfg.rope_theta, "rotary_dim": cfg.head_dim,
                                       "style": "rotate_half"})
        mixer = PartSpec(
            "softmax_attention",
            {"width": width, "n_heads": cfg.num_attention_heads,
             "n_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
             "scale": float(cfg.query_pre_attn_scalar) ** -0.5,
             "softcap": cfg.attn_logit_softcapping,
             "window": cfg.sliding_window if cfg.layer_is_sliding(l) else None,
             "position": position},
            {"q": p + "self_attn.q_proj.weight", "k": p + "self_attn.k_proj.weight",
             "v": p + "self_attn.v_proj.weight", "o": p + "self_attn.o_proj.weight"})
        ffn = PartSpec(
            "gated_mlp",
            {"width": width, "inner": cfg.intermediate_size, "activation": "gelu_tanh"},
            {"gate": p + "mlp.gate_proj.weight", "up": p + "mlp.up_proj.weight",
             "down": p + "mlp.down_proj.weight"})
        layers.append(LayerSpec(
            "sandwich", mixer, ffn,
            {"pre_mixer": norm(p + "input_layernorm.weight"),
             "post_mixer": norm(p + "post_attention_layernorm.weight"),
             "pre_ffn": norm(p + "pre_feedforward_layernorm.weight"),
             "post_ffn": norm(p + "post_feedforward_layernorm.weight")}))

    return ModelPlan(
        width=width,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("scaled_embedding",
                           {"vocab": cfg.vocab_size, "width": width, "scale": math.sqrt(width)},
                           {"table": "model.embed_tokens.weight"}),
        layers=layers,
        schedule=[LayerCall(l) for l in range(cfg.num_hidden_layers)],
        final_norm=norm("model.norm.weight"),
        head=PartSpec("linear_head",
                      {"vocab": cfg.vocab_size, "width": width,
                       "softcap": cfg.final_logit_softcapping},
                      {"table": "lm_head.weight", "tied_to": "model.embed_tokens.weight"}),
        stop_token_ids=tuple(cfg.eos_token_id),
    )


register_architecture("Gemma2ForCausalLM", Gemma2Config, gemma2_plan, model_type="gemma2")
