"""Qwen2ForCausalLM as a ``ModelSpec``: which parts, of which sizes, in which order.

The graph is that of v1/models/qwen2-7b/inference_fp16.dag:287-345 (one layer) and
:368-396 (the model); the tensor names are those that
v1/models/qwen2-7b/dump_from_huggingface.py:48-99 reads from the checkpoint.  QKV bias
is unconditional in this architecture (inference_fp16.dag:296,302,312)."""
from __future__ import annotations

from ..config.qwen2 import Qwen2Config
from ..config.registry import register_architecture
from ..parts.specs import (AttentionSpec, BlockSpec, EmbeddingSpec, GatedMLPSpec, HeadSpec, ModelSpec, NormSpec,
                           PositionSpec)


def qwen2_model_spec(cfg: Qwen2Config) -> ModelSpec:
    position = PositionSpec(kind="rotary", dim=cfg.head_dim, base=cfg.rope_theta,
                            max_positions=cfg.max_position_embeddings)
    norm = NormSpec(size=cfg.hidden_size, eps=cfg.rms_norm_eps)
    blocks = []
    for i in range(cfg.num_hidden_layers):
        blocks.append(BlockSpec(
            mixer=AttentionSpec(hidden=cfg.hidden_size, heads=cfg.num_attention_heads,
                                kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, qkv_bias=True,
                                out_bias=False, window=cfg.layer_window(i), position=position),
            ffn=GatedMLPSpec(hidden=cfg.hidden_size, inter=cfg.intermediate_size, activation=cfg.hidden_act),
            norm1=norm, norm2=norm, prefix=f"model.layers.{i}."))
    embedding = EmbeddingSpec(vocab=cfg.vocab_size, hidden=cfg.hidden_size, name="model.embed_tokens.weight")
    # the output head is a tensor of its own, or (tie_word_embeddings) the embedding's
    head = HeadSpec(vocab=cfg.vocab_size, hidden=cfg.hidden_size, norm=norm, norm_name="model.norm", name="lm_head.weight",
                    tied_to=embedding.name if cfg.tie_word_embeddings else None)
    return ModelSpec(vocab=cfg.vocab_size, hidden=cfg.hidden_size, blocks=tuple(blocks),
                     order=ModelSpec.default_order(len(blocks)), embedding=embedding, head=head,
                     max_positions=cfg.max_position_embeddings,
                     ignored=("*.rotary_emb.inv_freq",),      # older checkpoints store the rotation's frequencies
                     eos_token_ids=tuple(cfg.eos_token_id or ()))


register_architecture("Qwen2ForCausalLM", Qwen2Config, qwen2_model_spec, replace=True)
