"""Configuration and registry (no GPU)."""
import copy
import json
import os

import pytest

from llmgen_b200.config import ConfigError, Qwen3Config
from llmgen_b200.parts.registry import model_kernel_modules, model_weight_decls
from llmgen_b200.registry import (config_from_dict, config_from_folder, known_architectures, register_architecture,
                                  resolve, unregister_architecture)
from tests.util import TINY_A, TINY_B, TINY_C


def test_reads_every_key_of_the_architecture():
    arch, cfg = config_from_dict(TINY_B)
    assert arch.name == "Qwen3ForCausalLM" and isinstance(cfg, Qwen3Config)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers) == (384, 96, 320, 3)
    assert (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (8, 1, 32)
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 1e6 and cfg.max_position_embeddings == 256
    assert cfg.tie_word_embeddings is False
    assert cfg.layer_types == ("full_attention",) * 3 and cfg.sliding_window is None


def test_model_type_alone_names_the_architecture():
    d = {k: v for k, v in TINY_A.items() if k != "architectures"}
    arch, _ = config_from_dict(d)
    assert arch.name == "Qwen3ForCausalLM"


def test_head_dim_defaults_to_hidden_over_heads():
    d = {k: v for k, v in TINY_A.items() if k != "head_dim"}
    assert config_from_dict(d)[1].head_dim == 16


def test_missing_keys_are_all_listed():
    d = {k: v for k, v in TINY_A.items() if k not in ("rope_theta", "rms_norm_eps", "vocab_size")}
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    msg = str(e.value)
    assert "rope_theta" in msg and "rms_norm_eps" in msg and "vocab_size" in msg


@pytest.mark.parametrize("key,value,needle", [
    ("num_key_value_heads", 3, "multiple"),
    ("hidden_size", "64", "integer"),
    ("rms_norm_eps", 0, "> 0"),
    ("hidden_act", "gelu", "not supported"),
    ("attention_bias", True, "attention_bias"),
    ("rope_scaling", {"rope_type": "yarn", "factor": 4.0}, "rope_scaling"),
    ("layer_types", ["full_attention"], "layer_types"),
    ("head_dim", 15, "even"),
])
def test_bad_values_are_refused(key, value, needle):
    d = dict(TINY_A)
    d[key] = value
    with pytest.raises(ConfigError, match=needle):
        config_from_dict(d)


def test_window_layers():
    _, cfg = config_from_dict(TINY_C)
    assert cfg.sliding_window == 40
    assert cfg.layer_types == ("full_attention", "sliding_attention", "sliding_attention", "full_attention")
    d = {k: v for k, v in TINY_C.items() if k != "layer_types"}
    d["max_window_layers"] = 3
    _, cfg2 = config_from_dict(d)
    assert cfg2.layer_types == ("full_attention",) * 3 + ("sliding_attention",)
    d["use_sliding_window"] = False
    assert config_from_dict(d)[1].sliding_window is None
    d = dict(TINY_C)
    del d["sliding_window"]
    with pytest.raises(ConfigError, match="sliding_window"):
        config_from_dict(d)
    # the list of layer types stays in exported configurations whose switch is off: then no layer has a window
    off = dict(TINY_C, use_sliding_window=False)
    _, cfg3 = config_from_dict(off)
    assert cfg3.layer_types == ("full_attention",) * 4 and cfg3.sliding_window is None
    # without the switch the list decides
    unsaid = {k: v for k, v in TINY_C.items() if k != "use_sliding_window"}
    assert config_from_dict(unsaid)[1].layer_types == cfg.layer_types


def test_unknown_architecture():
    d = dict(TINY_A, architectures=["NoSuchModel"])
    with pytest.raises(ConfigError, match="unknown architecture.*Qwen3ForCausalLM"):
        config_from_dict(d)
    with pytest.raises(ConfigError, match="neither"):
        config_from_dict({"hidden_size": 4})


def test_spec_carries_every_size_as_a_parameter():
    arch, cfg = config_from_dict(TINY_C)
    spec = arch.build_spec(cfg)
    assert len(spec.layers) == 4 and [i.layer for i in spec.run_order] == [0, 1, 2, 3]
    a = spec.layers[1].mixer
    assert (a.num_heads, a.num_kv_heads, a.head_dim, a.window) == (6, 2, 48, 40)
    assert spec.layers[0].mixer.window is None
    assert abs(a.scale - 48 ** -0.5) < 1e-12 and a.position.theta == 50000.0 and a.q_norm.eps == 3e-6
    assert spec.layers[2].ffn.intermediate_size == 176 and not spec.tied
    names = {d.name for d in model_weight_decls(spec)}
    assert "lm_head.weight" in names and "model.layers.3.self_attn.k_norm.weight" in names
    assert len(names) == 3 + 4 * 11
    tied = arch.build_spec(config_from_dict(TINY_A)[1])
    assert tied.tied and "lm_head.weight" not in {d.name for d in model_weight_decls(tied)}
    assert "attention" in model_kernel_modules(spec)


def test_round_trip_through_a_folder(tmp_path):
    _, cfg = config_from_dict(TINY_C)
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    _, again = config_from_folder(str(tmp_path))
    assert again == cfg
    with pytest.raises(ConfigError, match="no such file"):
        config_from_folder(str(tmp_path / "nowhere"))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        config_from_folder(str(tmp_path))


def test_registering_another_architecture():
    class OtherConfig:
        @classmethod
        def from_dict(cls, data, where="config.json"):
            return cls()
    register_architecture("OtherForCausalLM", OtherConfig, lambda cfg: "spec", aliases=("other",))
    try:
        assert "OtherForCausalLM" in known_architectures()
        assert resolve("other").build_spec(None) == "spec"
        arch, cfg = config_from_dict({"model_type": "other"})
        assert isinstance(cfg, OtherConfig)
    finally:
        unregister_architecture("OtherForCausalLM")
    with pytest.raises(ConfigError):
        resolve("other")
