"""The Llama decoder as a description: RMSNorm, grouped-query attention with (llama3-scaled)
rotary encoding, SwiGLU feed-forward, in pre-norm blocks, final norm, LM head tied or not.

Parity: crates/model/src/llama.rs:142-170 (tensor names and assembly) of
akshajnad/rust_llm_inference_server.  This file holds no size: everything comes from LlamaConfig.
"""

from __future__ import annotations

from ..config.model_config import LlamaConfig
from ..config.registry import register_architecture
from ..parts.spec import (EmbeddingSpec, GQAAttentionSpec, LayerCall, LayerSpec, LMHeadSpec, ModelSpec,
                          RMSNormSpec, RopeSpec, SwiGLUSpec)


def describe_llama(cfg: LlamaConfig) -> ModelSpec:
    H, d = cfg.hidden_size, cfg.head_dim
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(LayerSpec(
            norm1=RMSNormSpec(H, cfg.rms_norm_eps, p + "input_layernorm.weight"),
            mixer=GQAAttentionSpec(
                hidden=H, n_heads=cfg.num_attention_heads, n_kv_heads=cfg.num_key_value_heads,
                head_dim=d, q_proj=p + "self_attn.q_proj.weight", k_proj=p + "self_attn.k_proj.weight",
                v_proj=p + "self_attn.v_proj.weight", o_proj=p + "self_attn.o_proj.weight",
                position=RopeSpec(d, cfg.rope_theta, cfg.rope_scaling)),
            norm2=RMSNormSpec(H, cfg.rms_norm_eps, p + "post_attention_layernorm.weight"),
            feed_forward=SwiGLUSpec(H, cfg.intermediate_size, p + "mlp.gate_proj.weight",
                                    p + "mlp.up_proj.weight", p + "mlp.down_proj.weight"),
        ))
    embed = "model.embed_tokens.weight"
    return ModelSpec(
        vocab_size=cfg.vocab_size, hidden=H,
        # the table's rows as they are (no scaling by sqrt(hidden), llama.rs:256-262)
        embedding=EmbeddingSpec(cfg.vocab_size, H, embed), layers=tuple(layers),
        order=tuple(LayerCall(i, i) for i in range(cfg.num_hidden_layers)),
        final_norm=RMSNormSpec(H, cfg.rms_norm_eps, "model.norm.weight"),
        # the product alone, in float32 (no logit scale, no cap, llama.rs:279-285)
        lm_head=LMHeadSpec(cfg.vocab_size, H, embed if cfg.tie_word_embeddings else "lm_head.weight"),
        max_positions=cfg.max_position_embeddings,
        # A tied checkpoint that still stores lm_head.weight is read without it
        # (crates/model/src/llama.rs:152-156).
        ignorable=("lm_head.weight",) if cfg.tie_word_embeddings else (),
        eos_token_ids=tuple(cfg.eos_token_ids),
    )


def llama_tensor_kinds(cfg: LlamaConfig) -> dict:
    """{name: (shape, "matrix" | "norm")} of every checkpoint tensor, for the random-weights mode."""
    H, d, I = cfg.hidden_size, cfg.head_dim, cfg.intermediate_size
    nh, nkv = cfg.num_attention_heads, cfg.num_key_value_heads
    out = {"model.embed_tokens.weight": ((cfg.vocab_size, H), "matrix"),
           "model.norm.weight": ((H,), "norm")}
    if not cfg.tie_word_embeddings:
        out["lm_head.weight"] = ((cfg.vocab_size, H), "matrix")
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        out[p + "input_layernorm.weight"] = ((H,), "norm")
        out[p + "post_attention_layernorm.weight"] = ((H,), "norm")
        out[p + "self_attn.q_proj.weight"] = ((nh * d, H), "matrix")
        out[p + "self_attn.k_proj.weight"] = ((nkv * d, H), "matrix")
        out[p + "self_attn.v_proj.weight"] = ((nkv * d, H), "matrix")
        out[p + "self_attn.o_proj.weight"] = ((H, nh * d), "matrix")
        out[p + "mlp.gate_proj.weight"] = ((I, H), "matrix")
        out[p + "mlp.up_proj.weight"] = ((I, H), "matrix")
        out[p + "mlp.down_proj.weight"] = ((H, I), "matrix")
    return out


register_architecture("LlamaForCausalLM", LlamaConfig.from_dict, describe_llama, llama_tensor_kinds)
