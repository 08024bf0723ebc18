"""The Qwen2.5 dense decoder as a list of parts.

Tensor names are the HuggingFace scheme that maeddesg/ROCmForge lists in src/config.rs:189-260;
the behaviours are its ``qwen2`` traits (src/config.rs:417-429): NeoX rotation, q/k/v bias,
no output-projection bias, theta and eps from the configuration.
"""
from __future__ import annotations

from ..config.qwen2 import Qwen2Config
from ..config.registry import register_architecture
from ..engine.model import ModelSpec, ScheduleEntry
from ..parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS
from ..parts.embedding import OutputHead, TokenEmbedding


def build_qwen2(cfg: Qwen2Config) -> ModelSpec:
    blocks, prefixes = [], []
    for layer in range(cfg.num_hidden_layers):
        position = POSITIONS.build("rope_neox", head_dim=cfg.head_dim, theta=cfg.rope_theta)
        mixer = MIXERS.build("gqa_attention", hidden=cfg.hidden_size, n_heads=cfg.num_attention_heads,
                             n_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, qkv_bias=True,
                             o_bias=False, window=cfg.window_of_layer(layer), position=position)
        ffn = FEED_FORWARDS.build("gated_mlp", hidden=cfg.hidden_size, intermediate=cfg.intermediate_size,
                                  activation=cfg.hidden_act)
        block = BLOCKS.build(
            "prenorm",
            norm1=NORMS.build("rmsnorm", size=cfg.hidden_size, eps=cfg.rms_norm_eps), mixer=mixer,
            norm2=NORMS.build("rmsnorm", size=cfg.hidden_size, eps=cfg.rms_norm_eps), ffn=ffn,
            names={"norm1": "input_layernorm.", "mixer": "self_attn.",
                   "norm2": "post_attention_layernorm.", "ffn": "mlp."})
        blocks.append(block)
        prefixes.append(f"model.layers.{layer}.")
    return ModelSpec(
        config=cfg,
        embedding=TokenEmbedding(cfg.vocab_size, cfg.hidden_size), embedding_prefix="model.embed_tokens.",
        blocks=blocks, block_prefixes=prefixes,
        final_norm=NORMS.build("rmsnorm", size=cfg.hidden_size, eps=cfg.rms_norm_eps),
        final_norm_prefix="model.norm.",
        head=OutputHead(cfg.vocab_size, cfg.hidden_size,
                        tied_to="model.embed_tokens.weight" if cfg.tie_word_embeddings else None),
        head_prefix="lm_head.",
        schedule=[ScheduleEntry(layer=i) for i in range(cfg.num_hidden_layers)],
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, max_position=cfg.max_position_embeddings,
        stop_token_ids=list(cfg.eos_token_ids),
    )


register_architecture(Qwen2Config.ARCHITECTURE, Qwen2Config, build_qwen2)
