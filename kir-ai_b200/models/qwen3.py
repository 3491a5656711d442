"""The Qwen3 dense decoder (``Qwen3ForCausalLM``) put together from parts.

Tensor names as the reference lists them (crates/llm-models/src/qwen.rs:215-300):
``model.embed_tokens.weight``, per layer ``input_layernorm``,
``self_attn.{q,k,v,o}_proj``, ``self_attn.{q,k}_norm``,
``post_attention_layernorm``, ``mlp.{gate,up,down}_proj``, then ``model.norm.weight``
and ``lm_head.weight`` (absent when ``tie_word_embeddings``).  Layer order,
norms and residuals: crates/llm-backend/src/core/qwen/ops/decoder.rs:210-314.
"""
from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..parts import Block, Embedding, GQAttention, OutputHead, RMSNorm, RotaryEmbedding, SwiGLU
from .plan import LayerCall, ModelPlan


def build_qwen3_plan(cfg: Qwen3Config) -> ModelPlan:
    blocks = []
    for layer in range(cfg.num_hidden_layers):
        base = f"model.layers.{layer}."
        attention = GQAttention(
            base + "self_attn.", cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
            RotaryEmbedding(cfg.head_dim, cfg.rope_theta),
            window=cfg.window_for_layer(layer), qk_norm_eps=cfg.rms_norm_eps,
        )
        blocks.append(Block(
            RMSNorm(base + "input_layernorm.weight", cfg.hidden_size, cfg.rms_norm_eps),
            attention,
            RMSNorm(base + "post_attention_layernorm.weight", cfg.hidden_size, cfg.rms_norm_eps),
            SwiGLU(base + "mlp.", cfg.hidden_size, cfg.intermediate_size),
            arrangement="pre_norm",
        ))
    head_name = "model.embed_tokens.weight" if cfg.tie_word_embeddings else "lm_head.weight"
    return ModelPlan(
        embedding=Embedding("model.embed_tokens.weight", cfg.vocab_size, cfg.hidden_size),
        blocks=blocks,
        order=[LayerCall(block=i, cache=i, write=True) for i in range(cfg.num_hidden_layers)],
        final_norm=RMSNorm("model.norm.weight", cfg.hidden_size, cfg.rms_norm_eps),
        head=OutputHead(head_name, cfg.vocab_size, cfg.hidden_size),
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        max_positions=cfg.max_position_embeddings,
        # some tied checkpoints still ship the head; the reference asks only for the names it needs and loads them
        ignorable_weights=["lm_head.weight"] if cfg.tie_word_embeddings else [],
    ).validate()
