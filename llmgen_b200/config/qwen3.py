"""Typed configuration of the Qwen3 dense decoder, read from its config.json keys.

Meaning of each field follows the reference's `qwen3.Config`
(src/models/qwen3.zig:74-140):

    num_hidden_layers        block_count
    hidden_size              embedding_length
    num_attention_heads      attention.head_count
    num_key_value_heads      attention.head_count_kv
    head_dim                 attention.key_length (decoupled from hidden/heads,
                             src/models/qwen3.zig:89-95)
    intermediate_size        feed_forward_length
    max_position_embeddings  context_length (rows of the rotary tables,
                             src/module/rope.zig:25)
    vocab_size               vocab_size
    rms_norm_eps             attention.layer_norm_rms_epsilon
    rope_theta               rope.rope_freq_base

`tie_word_embeddings` chooses between the embedding table and `lm_head.weight` for
the output projection (the reference hard-wires the tied case,
src/models/qwen3.zig:38).  The sliding-window keys of the architecture's config.json
(`sliding_window`, `use_sliding_window`, `max_window_layers`, `layer_types`) select,
layer by layer, between full causal attention and a causal window.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigReader

FULL_ATTENTION = "full_attention"
SLIDING_ATTENTION = "sliding_attention"


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    layer_types: Tuple[str, ...]
    sliding_window: Optional[int]
    hidden_act: str
    eos_token_ids: Tuple[int, ...]

    architecture = "Qwen3ForCausalLM"

    @classmethod
    def from_dict(cls, data: dict, where: str = "config.json") -> "Qwen3Config":
        r = ConfigReader(data, where)
        vocab = r.integer("vocab_size")
        hidden = r.integer("hidden_size")
        inter = r.integer("intermediate_size")
        layers = r.integer("num_hidden_layers")
        heads = r.integer("num_attention_heads")
        kv_heads = r.integer("num_key_value_heads", default=heads)
        head_dim = r.integer("head_dim", default=None)
        eps = r.number("rms_norm_eps")
        theta = r.number("rope_theta")
        max_pos = r.integer("max_position_embeddings")
        tie = r.boolean("tie_word_embeddings", default=False)
        act = r.string("hidden_act", default="silu", choices=("silu",))

        if head_dim is None and hidden is not None and heads is not None:
            if hidden % heads != 0:
                r.problem(f"'head_dim' is absent and hidden_size {hidden} is not a multiple of "
                          f"num_attention_heads {heads}")
            else:
                head_dim = hidden // heads
        if heads is not None and kv_heads is not None and heads % kv_heads != 0:
            r.problem(f"num_attention_heads {heads} must be a multiple of num_key_value_heads {kv_heads}")
        if head_dim is not None and head_dim % 2 != 0:
            r.problem(f"head_dim {head_dim} must be even (rotary pairs)")

        scaling = r.raw("rope_scaling")
        if scaling is not None:
            kind = scaling.get("rope_type", scaling.get("type")) if isinstance(scaling, dict) else scaling
            if kind not in (None, "default"):
                r.problem(f"'rope_scaling' of type {kind!r} is not supported")
        if r.raw("attention_bias", False) not in (False, None):
            r.problem("'attention_bias' = true is not supported (Qwen3 projections carry no bias)")

        # Which layers attend through a window.
        window = r.integer("sliding_window", default=None)
        use_window = r.boolean("use_sliding_window", default=None)
        layer_types = r.raw("layer_types")
        types: Tuple[str, ...] = ()
        if layers is not None:
            if layer_types is not None:
                if (not isinstance(layer_types, list) or len(layer_types) != layers
                        or any(t not in (FULL_ATTENTION, SLIDING_ATTENTION) for t in layer_types)):
                    r.problem(f"'layer_types' must list {layers} entries of "
                              f"'{FULL_ATTENTION}' or '{SLIDING_ATTENTION}'")
                elif use_window is False:
                    # the switch is off: every layer attends to all keys whatever the list and
                    # 'sliding_window' say (configurations are exported with the list left in place)
                    types = tuple(FULL_ATTENTION for _ in range(layers))
                else:
                    types = tuple(layer_types)
            elif use_window and window is not None:
                first_windowed = r.integer("max_window_layers", default=layers, minimum=0)
                if first_windowed is not None:
                    types = tuple(SLIDING_ATTENTION if i >= first_windowed else FULL_ATTENTION
                                  for i in range(layers))
            else:
                types = tuple(FULL_ATTENTION for _ in range(layers))
        if SLIDING_ATTENTION in types and window is None:
            r.problem("a layer of type 'sliding_attention' needs 'sliding_window'")
        if SLIDING_ATTENTION not in types:
            window = None

        eos_raw = r.raw("eos_token_id")
        eos: Tuple[int, ...] = ()
        if isinstance(eos_raw, int) and not isinstance(eos_raw, bool):
            eos = (eos_raw,)
        elif isinstance(eos_raw, list) and all(isinstance(e, int) for e in eos_raw):
            eos = tuple(eos_raw)
        elif eos_raw is not None:
            r.problem(f"'eos_token_id' must be an integer or a list of integers, got {eos_raw!r}")
        r.finish()
        return cls(vocab_size=vocab, hidden_size=hidden, intermediate_size=inter,
                   num_hidden_layers=layers, num_attention_heads=heads,
                   num_key_value_heads=kv_heads, head_dim=head_dim, rms_norm_eps=eps,
                   rope_theta=theta, max_position_embeddings=max_pos, tie_word_embeddings=tie,
                   layer_types=types, sliding_window=window, hidden_act=act, eos_token_ids=eos)

    def to_dict(self) -> dict:
        """The config.json form of this configuration (what the random-weights mode writes)."""
        d = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": self.hidden_act,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "attention_bias": False,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
        }
        if self.sliding_window is not None:
            d["sliding_window"] = self.sliding_window
            d["use_sliding_window"] = True
            d["layer_types"] = list(self.layer_types)
        else:
            d["sliding_window"] = None
            d["use_sliding_window"] = False
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        return d
