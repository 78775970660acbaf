"""The Qwen2.5 dense decoder ("Qwen2ForCausalLM") as the reference computes it
(pyre/model.py): pre-norm blocks of RMSNorm, grouped-query attention with biased
q/k/v and unbiased o projections and half-split rotary, SwiGLU feed-forward; final
RMSNorm; linear head, optionally tied to the embedding.

This file only turns the configuration into a ModelSpec, layer by layer; all the
computing is in ``pyre_b200.parts``.
"""

from __future__ import annotations

from ..config.model_config import Qwen2Config
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .spec import ModelSpec


def build_qwen2(cfg: Qwen2Config) -> ModelSpec:
    def norm():
        return PartSpec("rms_norm", {"width": cfg.hidden_size, "eps": cfg.rms_norm_eps})

    blocks = []
    for _layer in range(cfg.num_hidden_layers):
        mixer = PartSpec("attention", {
            "width": cfg.hidden_size, "n_heads": cfg.num_attention_heads,
            "n_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "qkv_bias": True, "o_bias": False, "window": None,
            "position": PartSpec("rotary", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta}),
        })
        ffn = PartSpec("gated_mlp", {"width": cfg.hidden_size, "intermediate": cfg.intermediate_size,
                                     "activation": "silu"})
        blocks.append(PartSpec("prenorm", {"norm1": norm(), "mixer": mixer, "norm2": norm(), "ffn": ffn}))
    return ModelSpec(
        embed=PartSpec("token_embedding", {"vocab": cfg.vocab_size, "width": cfg.hidden_size}),
        blocks=blocks,
        final_norm=norm(),
        head=PartSpec("linear_head", {"vocab": cfg.vocab_size, "width": cfg.hidden_size,
                                      "tied_to": "model.embed_tokens.weight" if cfg.tie_word_embeddings else None}),
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
    )


register_architecture(Qwen2Config.architecture, Qwen2Config, build_qwen2)
