"""Gemma-2 as data: its configuration turned into a :class:`ModelSpec`.

Nothing here computes.  This file only says which parts a Gemma-2 layer is made
of, with which constants, and what its tensors are called in the weight file.

Formulas, in the order the reference computes them (runtime/src/lib.rs:4527-4540,
4553-4561): ``h = E[id]*sqrt(hidden)``; per layer
``h += post_attention_norm(attn(input_norm(h)))`` and
``h += post_feedforward_norm(mlp(pre_feedforward_norm(h)))``; logits from
``final_norm(h)`` through the tied embedding, then the final soft cap.  All norms
are of the ``(1+w)`` form (model/export_gemma.py:25-26 adds the 1 at export).
Attention: no bias, rotate-half RoPE, tanh soft cap on the scaled scores
(runtime/cuda/codebook_gemv.cu:219-230, 250-255).  The reference scales by
``rsqrt(head_dim)`` and refuses other values of ``query_pre_attn_scalar``
(model/export_gemma.py:46-47) and does not model the sliding window
(runtime/src/lib.rs:4455); here both are parameters of the attention part.
"""
from __future__ import annotations

import math

from ..config.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
from ..config.gemma2 import Gemma2Config


def gemma2_spec(cfg: Gemma2Config) -> ModelSpec:
    H = cfg.hidden_size

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": H, "eps": cfg.rms_norm_eps, "unit_offset": True, "weight": name})

    layers = []
    for i in range(cfg.num_hidden_layers):
        window = cfg.sliding_window if cfg.is_sliding(i) else None
        mixer = PartSpec("attention", {
            "hidden_size": H,
            "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim,
            "scale": cfg.attention_scale,
            "softcap": cfg.attn_logit_softcapping,
            "window": window,
            "position": PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta,
                                          "rotary_dim": cfg.head_dim}),
            "q": "self_attn.q_proj.weight", "k": "self_attn.k_proj.weight",
            "v": "self_attn.v_proj.weight", "o": "self_attn.o_proj.weight",
        })
        ffn = PartSpec("gated_mlp", {
            "hidden_size": H,
            "intermediate_size": cfg.intermediate_size,
            "activation": "gelu_tanh",
            "gate": "mlp.gate_proj.weight", "up": "mlp.up_proj.weight", "down": "mlp.down_proj.weight",
        })
        block = PartSpec("sandwich", {
            "pre_mixer_norm": norm("input_layernorm.weight"),
            "post_mixer_norm": norm("post_attention_layernorm.weight"),
            "pre_ffn_norm": norm("pre_feedforward_layernorm.weight"),
            "post_ffn_norm": norm("post_feedforward_layernorm.weight"),
        })
        layers.append(LayerSpec(block=block, mixer=mixer, feed_forward=ffn, prefix=f"model.layers.{i}."))

    return ModelSpec(
        architecture="Gemma2ForCausalLM",
        hidden_size=H,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("embedding", {"vocab_size": cfg.vocab_size, "hidden_size": H,
                                         "scale": math.sqrt(H), "weight": "model.embed_tokens.weight"}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=norm("model.norm.weight"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": H,
                                      "softcap": cfg.final_logit_softcapping,
                                      "weight": "lm_head.weight",
                                      "tied_to": "model.embed_tokens.weight" if cfg.tie_word_embeddings else None}),
        max_positions=cfg.max_position_embeddings,
        stop_ids=cfg.eos_token_id,
    )


register_architecture("Gemma2ForCausalLM", Gemma2Config, gemma2_spec)
