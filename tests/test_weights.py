"""Weights by name: reading, checking, random folders (no GPU)."""
import json
import os
import struct

import pytest
import torch
from safetensors.torch import load_file, save_file

from llmgen_b200.engine.api import write_random_model
from llmgen_b200.parts.registry import model_weight_decls
from llmgen_b200.parts.spec import INT_TABLE, WeightDecl
from llmgen_b200.registry import config_from_dict
from llmgen_b200.weights import (TensorDirectory, WeightError, open_weights, random_tensors, weights_from_dict,
                                 write_safetensors)
from tests.util import TINY, TINY_A, TINY_B, make_folder


def _decls(cfg):
    arch, c = config_from_dict(cfg)
    return model_weight_decls(arch.build_spec(c))


def test_random_folder_is_readable_by_the_safetensors_library(tmp_path):
    path = make_folder(str(tmp_path), "A")
    assert sorted(os.listdir(path)) == ["config.json", "model.safetensors"]
    theirs = load_file(os.path.join(path, "model.safetensors"))
    ours = TensorDirectory(path)
    assert set(theirs) == set(ours.names()) == {d.name for d in _decls(TINY_A)}
    for name, t in theirs.items():
        assert t.dtype == torch.bfloat16
        assert torch.equal(ours.tensor(name), t)
    cfg = json.load(open(os.path.join(path, "config.json")))
    assert cfg["architectures"] == ["Qwen3ForCausalLM"] and cfg["head_dim"] == 16


def test_reader_reads_what_the_library_wrote(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int64).view(2, 3)}
    save_file(tensors, str(tmp_path / "model.safetensors"))
    d = TensorDirectory(str(tmp_path))
    for k, v in tensors.items():
        assert torch.equal(d.tensor(k), v) and d.entry(k).shape == tuple(v.shape)


def test_seed_and_statistics(tmp_path):
    decls = _decls(TINY_B)
    a = random_tensors(decls, 1, 0.03, 0.05, torch.float32)
    b = random_tensors(decls, 1, 0.03, 0.05, torch.float32)
    c = random_tensors(decls, 2, 0.03, 0.05, torch.float32)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    w = a["model.layers.0.mlp.gate_proj.weight"]
    assert abs(float(w.mean())) < 2e-3 and abs(float(w.std()) - 0.03) < 2e-3
    g = a["model.layers.1.self_attn.q_norm.weight"]
    assert abs(float(g.mean()) - 1.0) < 0.05 and g.shape == (32,)
    # a tensor's values do not depend on which other tensors exist
    only = random_tensors([d for d in decls if d.name == "model.norm.weight"], 1, 0.03, 0.05, torch.float32)
    assert torch.equal(only["model.norm.weight"], a["model.norm.weight"])


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    path = make_folder(str(tmp_path), "A")
    f = os.path.join(path, "model.safetensors")
    t = load_file(f)
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 63, dtype=torch.bfloat16)
    t["rotary.inv_freq"] = torch.zeros(8)
    t["model.layers.0.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)
    save_file(t, f)
    with pytest.raises(WeightError) as e:
        open_weights(path, _decls(TINY_A))
    msg = str(e.value)
    assert "missing (2)" in msg and "model.layers.1.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "unexpected (1)" in msg and "rotary.inv_freq" in msg
    assert "[64, 63]" in msg and "[64, 64]" in msg
    assert "dtype I32" in msg


def _spec(cfg):
    arch, c = config_from_dict(cfg)
    return arch.build_spec(c)


def test_untied_model_needs_lm_head_and_tied_takes_only_a_true_copy(tmp_path):
    path = make_folder(str(tmp_path), "B")
    f = os.path.join(path, "model.safetensors")
    t = load_file(f)
    head = t.pop("lm_head.weight")
    save_file(t, f)
    with pytest.raises(WeightError, match="missing.*lm_head.weight"):
        open_weights(path, _decls(TINY_B))
    path_a = make_folder(str(tmp_path), "A")
    fa = os.path.join(path_a, "model.safetensors")
    ta = {k: v.clone() for k, v in load_file(fa).items()}     # copies: the file these came from is written again below
    ta["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)
    save_file(ta, fa)
    with pytest.raises(WeightError, match="unexpected.*lm_head.weight"):
        open_weights(path_a, _decls(TINY_A))               # nothing said that it may be there
    # exports of tied models often carry the output matrix too: the architecture lets it pass if it is the
    # table's copy (and rotary buffers whatever they hold), and still refuses anything else
    spec = _spec(TINY_A)
    with pytest.raises(WeightError, match="lm_head.weight.*differ"):
        open_weights(path_a, _decls(TINY_A), spec.ignorable_tensors, spec.same_as)
    ta["lm_head.weight"] = ta["model.embed_tokens.weight"].clone()
    ta["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(8)
    save_file(ta, fa)
    store = open_weights(path_a, _decls(TINY_A), spec.ignorable_tensors, spec.same_as)
    assert torch.equal(store.host_tensor("model.embed_tokens.weight"), ta["model.embed_tokens.weight"])
    with pytest.raises(WeightError, match="not declared"):
        store.host_tensor("lm_head.weight")
    ta["stray.weight"] = torch.ones(3)
    save_file(ta, fa)
    with pytest.raises(WeightError, match=r"unexpected \(1\): stray.weight"):
        open_weights(path_a, _decls(TINY_A), spec.ignorable_tensors, spec.same_as)


def test_broken_files(tmp_path):
    with pytest.raises(WeightError, match="no model.safetensors"):
        open_weights(str(tmp_path), _decls(TINY_A))
    f = tmp_path / "model.safetensors"
    f.write_bytes(b"\x01\x02")
    with pytest.raises(WeightError, match="truncated"):
        open_weights(str(tmp_path), _decls(TINY_A))
    f.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(WeightError, match="header length"):
        open_weights(str(tmp_path), _decls(TINY_A))
    header = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    f.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 8)
    with pytest.raises(WeightError, match="needs 16 bytes"):
        open_weights(str(tmp_path), _decls(TINY_A))


def test_dtypes_kept_as_the_rules_say():
    decls = [WeightDecl("m", (4, 4)), WeightDecl("v", (4,), "vector"), WeightDecl("i", (3,), INT_TABLE)]
    store = weights_from_dict({"m": torch.randn(4, 4).to(torch.bfloat16), "v": torch.ones(4, dtype=torch.bfloat16),
                               "i": torch.tensor([1, 2, 3], dtype=torch.int64)}, decls)
    assert store.device_tensor("m", torch.bfloat16, "cpu").dtype == torch.bfloat16
    assert store.device_tensor("m", torch.float32, "cpu").dtype == torch.float32      # the 32-bit path widens
    assert store.device_tensor("v", torch.bfloat16, "cpu").dtype == torch.float32     # vectors are float32
    assert store.device_tensor("i", torch.bfloat16, "cpu").dtype == torch.int32       # integer tables int32
    assert store.device_tensor("m", torch.bfloat16, "cpu") is store.device_tensor("m", torch.bfloat16, "cpu")
    with pytest.raises(WeightError, match="not declared"):
        store.device_tensor("zzz", torch.float32, "cpu")
    with pytest.raises(WeightError, match="declared with shapes"):
        weights_from_dict({}, [WeightDecl("m", (4, 4)), WeightDecl("m", (4, 5))])


def test_sharded_folder(tmp_path):
    write_safetensors(str(tmp_path / "s1.safetensors"), {"a": torch.ones(2, 2)})
    write_safetensors(str(tmp_path / "s2.safetensors"), {"b": torch.zeros(3)})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    d = TensorDirectory(str(tmp_path))
    assert sorted(d.names()) == ["a", "b"] and float(d.tensor("a").sum()) == 4.0
