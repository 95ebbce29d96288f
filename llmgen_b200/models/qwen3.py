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
from typing import Dict, List

from ..config.qwen3 import SLIDING_ATTENTION, Qwen3Config
from ..parts.spec import (AttentionSpec, GatedMLPSpec, ModelSpec, PreNormBlockSpec, RMSNormSpec,
                          RopeSpec, default_run_order)
from ..registry import register_architecture
from ..weights.gguf import GGUFError, register_gguf_source


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
        max_positions=cfg.max_position_embeddings, eos_token_ids=cfg.eos_token_ids,
        # exports of tied models often still carry the output matrix (a copy of the table), and some carry the
        # rotary inverse frequencies as a buffer: neither is read, the copy must be one
        ignorable_tensors=(("lm_head.weight",) if cfg.tie_word_embeddings else ()) + ("*.rotary_emb.inv_freq",),
        same_as=(("lm_head.weight", embedding),) if cfg.tie_word_embeddings else ())


register_architecture("Qwen3ForCausalLM", Qwen3Config, build_qwen3_spec, aliases=("qwen3",))


# ------------------------------------------------------------------ the reference's model files
# the reference's names (left, `.weight` appended) and this engine's (right)
_GLOBAL_NAMES = {"token_embd": "model.embed_tokens", "output_norm": "model.norm"}
_LAYER_NAMES = {
    "attn_norm": "input_layernorm", "attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj",
    "attn_output": "self_attn.o_proj", "attn_q_norm": "self_attn.q_norm", "attn_k_norm": "self_attn.k_norm",
    "ffn_norm": "post_attention_layernorm", "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj",
}
GGUF_ARCHITECTURE = "qwen3"      # `general.architecture` of the reference's files


def gguf_config(g) -> dict:
    """config.json of the Qwen3 model a GGUF file describes, from the metadata keys the reference reads
    (src/models/qwen3.zig:100-140); one error lists every key that is missing."""
    arch = GGUF_ARCHITECTURE
    meta, missing = g.metadata, []

    def need(*names):
        for name in names:
            if f"{arch}.{name}" in meta:
                return meta[f"{arch}.{name}"]
        missing.append(" or ".join(f"{arch}.{n}" for n in names))
        return 0

    vocab = meta.get(f"{arch}.vocab_size") or len(meta.get("tokenizer.ggml.tokens") or ())
    if not vocab and "token_embd.weight" in g.tensors:
        vocab = g.tensors["token_embd.weight"].shape[0]
    if not vocab:
        missing.append(f"{arch}.vocab_size (or tokenizer.ggml.tokens)")
    heads = need("attention.head_count")
    hidden = need("embedding_length")
    cfg = {
        "architectures": [Qwen3Config.architecture], "model_type": arch,
        "vocab_size": int(vocab), "hidden_size": int(hidden), "intermediate_size": int(need("feed_forward_length")),
        "num_hidden_layers": int(need("block_count")), "num_attention_heads": int(heads),
        "num_key_value_heads": int(meta.get(f"{arch}.attention.head_count_kv", heads)),
        "rms_norm_eps": float(meta.get(f"{arch}.attention.layer_norm_rms_epsilon", 1e-6)),
        "rope_theta": float(need("rope.freq_base", "rope.rope_freq_base")),
        "max_position_embeddings": int(need("context_length")),
        "tie_word_embeddings": "output.weight" not in g.tensors, "hidden_act": "silu",
    }
    if f"{arch}.attention.key_length" in meta:
        cfg["head_dim"] = int(meta[f"{arch}.attention.key_length"])
        value_length = meta.get(f"{arch}.attention.value_length", cfg["head_dim"])
        if int(value_length) != cfg["head_dim"]:
            raise GGUFError(f"{g.path}: key_length {cfg['head_dim']} and value_length {value_length} differ")
    eos = meta.get("tokenizer.ggml.eos_token_id")
    if isinstance(eos, int) and eos >= 0:
        cfg["eos_token_id"] = eos
    if missing:
        raise GGUFError(f"{g.path}: metadata keys are missing: " + "; ".join(missing))
    return cfg


def gguf_tensor_names(g, cfg: dict) -> Dict[str, str]:
    """This engine's tensor name for every tensor of the file (the reference's table, src/models/qwen3.zig:34-55);
    unknown names are an error."""
    num_layers = cfg["num_hidden_layers"]
    out: Dict[str, str] = {}
    unknown: List[str] = []
    for name in g.tensors:
        stem, dot, last = name.rpartition(".")
        parts = stem.split(".")
        if last != "weight" or not dot:
            unknown.append(name)
        elif stem == "output":
            out[name] = "lm_head.weight"
        elif stem in _GLOBAL_NAMES:
            out[name] = _GLOBAL_NAMES[stem] + ".weight"
        elif len(parts) == 3 and parts[0] == "blk" and parts[1].isdigit() and parts[2] in _LAYER_NAMES \
                and int(parts[1]) < num_layers:
            out[name] = f"model.layers.{int(parts[1])}.{_LAYER_NAMES[parts[2]]}.weight"
        else:
            unknown.append(name)
    if unknown:
        raise GGUFError(f"{g.path}: tensors with no place in the model ({len(unknown)}): " + ", ".join(sorted(unknown)[:20]))
    return out


register_gguf_source(GGUF_ARCHITECTURE, gguf_config, gguf_tensor_names)
