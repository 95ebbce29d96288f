"""Qwen3 dense: from its typed configuration to a `ModelSpec`.

Layer arrangement and tensor roles follow the reference's model
(src/models/qwen3.zig:142-340) and its name table `STATE_DCIT`
(src/models/qwen3.zig:34-68); the tensor names are those of a safetensors model folder:

    token_embd        model.embed_tokens.weight            [vocab, hidden]
    output_norm       model.norm.weight                    [hidden]
    (untied only)     lm_head.weight                       [vocab, hidden]
    attn_norm         model.layers.L.input_layernorm.weight
    attn_q/k/v        model.layers.L.self_attn.{q,k,v}_proj.weight   [out, in]
    attn_q/k_norm     model.layers.L.self_attn.{q,k}_norm.weight     [head_dim]
    attn_output       model.layers.L.self_attn.o_proj.weight
    ffn_norm          model.layers.L.post_attention_layernorm.weight
    ffn_gate/up/down  model.layers.L.mlp.{gate,up,down}_proj.weight

Fixed by the architecture, not by its config.json: scale = 1/sqrt(head_dim)
(src/executor.zig:877), causal attention, no biases, half-split rotary pairing over the
whole head, SiLU gate, pre-norm residual layout.
"""
from __future__ import annotations

import math

from ..config.qwen3 import SLIDING_ATTENTION, Qwen3Config
from ..parts.spec import (AttentionSpec, GatedMLPSpec, ModelSpec, PreNormBlockSpec, RMSNormSpec,
                          RopeSpec, default_run_order)
from ..registry import register_architecture


def build_qwen3_spec(cfg: Qwen3Config) -> ModelSpec:
    rope = RopeSpec(rotary_dim=cfg.head_dim, theta=cfg.rope_theta, max_positions=cfg.max_position_embeddings)
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        windowed = cfg.layer_types[i] == SLIDING_ATTENTION
        attn = AttentionSpec(
            hidden_size=cfg.hidden_size, num_heads=cfg.num_attention_heads,
            num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
            scale=1.0 / math.sqrt(cfg.head_dim),
            q_proj=p + "self_attn.q_proj.weight", k_proj=p + "self_attn.k_proj.weight",
            v_proj=p + "self_attn.v_proj.weight", o_proj=p + "self_attn.o_proj.weight",
            q_norm=RMSNormSpec(cfg.head_dim, cfg.rms_norm_eps, p + "self_attn.q_norm.weight"),
            k_norm=RMSNormSpec(cfg.head_dim, cfg.rms_norm_eps, p + "self_attn.k_norm.weight"),
            position=rope, window=cfg.sliding_window if windowed else None)
        mlp = GatedMLPSpec(
            hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
            gate_proj=p + "mlp.gate_proj.weight", up_proj=p + "mlp.up_proj.weight",
            down_proj=p + "mlp.down_proj.weight", activation=cfg.hidden_act)
        layers.append(PreNormBlockSpec(
            mixer_norm=RMSNormSpec(cfg.hidden_size, cfg.rms_norm_eps, p + "input_layernorm.weight"),
            mixer=attn,
            ffn_norm=RMSNormSpec(cfg.hidden_size, cfg.rms_norm_eps, p + "post_attention_layernorm.weight"),
            ffn=mlp))
    embedding = "model.embed_tokens.weight"
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
        embedding=embedding, layers=tuple(layers), run_order=default_run_order(cfg.num_hidden_layers),
        final_norm=RMSNormSpec(cfg.hidden_size, cfg.rms_norm_eps, "model.norm.weight"),
        lm_head=embedding if cfg.tie_word_embeddings else "lm_head.weight",
        max_positions=cfg.max_position_embeddings, eos_token_ids=cfg.eos_token_ids)


register_architecture("Qwen3ForCausalLM", Qwen3Config, build_qwen3_spec, aliases=("qwen3",))
