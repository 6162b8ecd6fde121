"""Qwen2ForCausalLM as a blueprint of parts.

The dense GQA decoder of ``engine/model.py`` in davidjoyme/flashdecode-cuda:
token embedding; per layer RMSNorm -> attention with q/k/v bias and rotate-half
rotary encoding -> RMSNorm -> SiLU-gated feed-forward, both with a residual
add; final RMSNorm; output head that is the embedding table when the
configuration ties them.  Tensor names are the checkpoint's own
(engine/model.py:100,166,175-232; engine/loader.py:52-67).
"""

from __future__ import annotations

from ..config.qwen2 import Qwen2Config
from ..engine.blueprint import LayerSpec, ModelBlueprint, PartSpec, RunSpec
from ..registry import register_architecture


def qwen2_blueprint(cfg: Qwen2Config) -> ModelBlueprint:
    H = cfg.hidden_size
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        layers.append(LayerSpec(
            block="prenorm",
            norm1=PartSpec("norm", "rmsnorm", dict(size=H, eps=cfg.rms_norm_eps), f"{p}.input_layernorm"),
            mixer=PartSpec("mixer", "gqa_attention",
                           dict(hidden_size=H, n_heads=cfg.num_attention_heads,
                                n_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
                                position="rope", window=cfg.layer_window(i), bias=cfg.attention_bias),
                           f"{p}.self_attn"),
            norm2=PartSpec("norm", "rmsnorm", dict(size=H, eps=cfg.rms_norm_eps), f"{p}.post_attention_layernorm"),
            feed_forward=PartSpec("feed_forward", "swiglu",
                                  dict(hidden_size=H, intermediate_size=cfg.intermediate_size), f"{p}.mlp"),
        ))
    return ModelBlueprint(
        hidden_size=H,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("embedding", "token_table", dict(vocab_size=cfg.vocab_size, hidden_size=H),
                           "model.embed_tokens"),
        positions={"rope": PartSpec("position", "rotary_half",
                                    dict(head_dim=cfg.head_dim, theta=cfg.rope_theta,
                                         max_positions=cfg.max_position_embeddings))},
        layers=layers,
        schedule=[RunSpec(i) for i in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("norm", "rmsnorm", dict(size=H, eps=cfg.rms_norm_eps), "model.norm"),
        head=PartSpec("head", "linear_head",
                      dict(vocab_size=cfg.vocab_size, hidden_size=H,
                           tied_to="model.embed_tokens.weight" if cfg.tie_word_embeddings else None),
                      "lm_head"),
        max_positions=cfg.max_position_embeddings,
    )


register_architecture("Qwen2ForCausalLM", Qwen2Config, qwen2_blueprint)
