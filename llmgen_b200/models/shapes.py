"""Configurations of published Qwen3 dense sizes, for runs with random weights (benchmarks and `--random NAME`).

The sizes are the architecture's public config.json values; no weights come with them.
"""
from __future__ import annotations

_COMMON = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_key_value_heads": 8, "head_dim": 128,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 40960, "hidden_act": "silu",
}
QWEN3_SHAPES = {
    "qwen3-0.6b": dict(_COMMON, num_hidden_layers=28, hidden_size=1024, num_attention_heads=16, intermediate_size=3072,
                       tie_word_embeddings=True),
    "qwen3-8b": dict(_COMMON, num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, intermediate_size=12288,
                     tie_word_embeddings=False),
    "qwen3-32b": dict(_COMMON, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600,
                      tie_word_embeddings=False),
}


def named_shape(name: str) -> dict:
    try:
        return dict(QWEN3_SHAPES[name.lower()])
    except KeyError:
        raise ValueError(f"unknown shape {name!r}; known: {', '.join(sorted(QWEN3_SHAPES))}") from None
