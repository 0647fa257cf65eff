"""The Qwen3 dense decoder (``Qwen3ForCausalLM``), put together from the package's parts.

Per layer, in the reference's order (src/model/mod.rs:645-650): input RMSNorm, grouped-query
attention with per-head q/k RMSNorm and rotary embedding (src/model/attention.rs:868-914),
residual, post-attention RMSNorm, SwiGLU feed-forward (src/model/layers.rs:625-648), residual;
then the final RMSNorm and the head, tied to the embedding or not (src/model/mod.rs:723-761).
Tensor names are the checkpoint's own, under ``model.`` (src/model/mod.rs:244-321).
"""
from __future__ import annotations

import torch

from ..config.qwen3 import FULL_ATTENTION, Qwen3Config
from ..config.registry import register_architecture
from ..parts.block import PreNormBlock
from ..parts.embedding import Embedding, LMHead
from ..parts.model import DecoderModel
from ..parts.registry import build_part


def build_qwen3(cfg: Qwen3Config, max_positions: int) -> DecoderModel:
    position = build_part("position", "rotary", head_dim=cfg.head_dim, theta=cfg.rope_theta,
                          max_positions=max_positions, scaling=cfg.rope_scaling)
    blocks = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        kind = cfg.layer_types[i]
        mixer = build_part("mixer", kind, hidden=cfg.hidden_size, heads=cfg.num_attention_heads,
                           kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, prefix=f"{p}.self_attn",
                           position=position, qk_norm_eps=cfg.rms_norm_eps,
                           window=0 if kind == FULL_ATTENTION else cfg.sliding_window)
        ffn = build_part("feed_forward", "gated_mlp", hidden=cfg.hidden_size, intermediate=cfg.intermediate_size,
                         prefix=f"{p}.mlp", activation=cfg.hidden_act)
        blocks.append(PreNormBlock(
            build_part("norm", "rmsnorm", width=cfg.hidden_size, eps=cfg.rms_norm_eps, name=f"{p}.input_layernorm.weight"),
            mixer,
            build_part("norm", "rmsnorm", width=cfg.hidden_size, eps=cfg.rms_norm_eps,
                       name=f"{p}.post_attention_layernorm.weight"),
            ffn))
    embedding = Embedding(cfg.vocab_size, cfg.hidden_size, "model.embed_tokens.weight")
    final_norm = build_part("norm", "rmsnorm", width=cfg.hidden_size, eps=cfg.rms_norm_eps, name="model.norm.weight")
    if cfg.tie_word_embeddings:
        head = LMHead(cfg.vocab_size, cfg.hidden_size, final_norm, None, tied_to=embedding,
                      redundant_name="lm_head.weight")
    else:
        head = LMHead(cfg.vocab_size, cfg.hidden_size, final_norm, "lm_head.weight")
    return DecoderModel(cfg, embedding, blocks, head)


register_architecture("Qwen3ForCausalLM", Qwen3Config.from_dict, build_qwen3, model_types=("qwen3",), replace=True)
