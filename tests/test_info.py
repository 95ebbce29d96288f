"""`python -m llmgen_b200 info`: what a model folder holds, checked without a GPU."""
import json
import os
import subprocess
import sys

import pytest
import torch

from tests.util import ROOT, TINY_A, TINY_C

from llmgen_b200.engine.api import write_random_model
from llmgen_b200.info import describe
from llmgen_b200.weights.loader import WeightError
from llmgen_b200.weights.safetensors_io import SafetensorsFile, write_safetensors


def test_describe_names_every_size_and_groups_equal_layers():
    text = describe(config=TINY_C, context=100)
    first = text.splitlines()[0]
    for piece in ("Qwen3ForCausalLM", "layers=4", "hidden=80", "heads=6/2", "head_dim=48", "eps=3e-06", "rope=50000",
                  "ffn=176", "vocab=301", "positions=768", "untied"):
        assert piece in first, piece
    assert "  layer 0: attention 6/2 heads x 48, all keys" in text
    assert "  layers 1-2: attention 6/2 heads x 48, window 40" in text and "  layer 3: " in text
    # embedding + lm_head + 4 x (q, k, v, o, gate, up, down) matrices; 2 gains a head norm pair, 2 a layer, 1 final
    per_layer = 80 * 288 + 2 * 80 * 96 + 288 * 80 + 3 * 80 * 176
    matrices = 2 * 301 * 80 + 4 * per_layer
    assert f"{matrices:,} in matrices" in text and f"{matrices + 4 * (2 * 80 + 2 * 48) + 80:,} values" in text
    assert f"in matrix products per token: {4 * per_layer + 301 * 80:,} weights" in text
    assert f"cache: {4 * 2 * 96 * 2:,} bytes per token" in text and "for 100 tokens" in text
    assert "model file" not in text                           # a configuration alone has no file to check


def test_describe_checks_the_tensors_of_a_folder(tmp_path):
    path = write_random_model(str(tmp_path / "a"), TINY_A, seed=0)
    text = describe(model_dir=path)
    assert "layers 0-1: attention 4/2 heads x 16, all keys" in text and "tied output projection" in text
    assert "model file: every declared tensor is there with its shape (24 stored as BF16)" in text
    # a folder with config.json only
    bare = tmp_path / "bare"
    bare.mkdir()
    with open(bare / "config.json", "w", encoding="utf-8") as f:
        json.dump(TINY_A, f)
    assert "model file: none in the folder" in describe(model_dir=str(bare))
    # a tensor with another shape, one too many, one missing: all in one error
    file = os.path.join(path, "model.safetensors")
    stored = SafetensorsFile(file)
    tensors = {name: stored.tensor(name).clone() for name in stored.entries}
    del stored
    tensors["model.norm.weight"] = torch.zeros(3)
    tensors["extra.weight"] = torch.zeros(2, 2)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    write_safetensors(file, tensors)
    with pytest.raises(WeightError) as err:
        describe(model_dir=path)
    for piece in ("model.norm.weight", "extra.weight", "model.layers.1.mlp.up_proj.weight"):
        assert piece in str(err.value)


def test_info_command(tmp_path):
    path = write_random_model(str(tmp_path / "c"), TINY_C, seed=5)
    env = dict(os.environ, PYTHONPATH=ROOT)
    ok = subprocess.run([sys.executable, "-m", "llmgen_b200", "info", "--model", path, "--max-model-len", "512"],
                        env=env, capture_output=True, text=True, timeout=300)
    assert ok.returncode == 0, ok.stderr
    assert "layers 1-2: attention 6/2 heads x 48, window 40" in ok.stdout and "for 512 tokens" in ok.stdout
    assert "model file: every declared tensor is there" in ok.stdout
    cfg = tmp_path / "bad.json"
    cfg.write_text(json.dumps({k: v for k, v in TINY_C.items() if k not in ("rope_theta", "vocab_size")}))
    bad = subprocess.run([sys.executable, "-m", "llmgen_b200", "info", "--random", str(cfg)], env=env,
                         capture_output=True, text=True, timeout=300)
    assert bad.returncode == 1 and "rope_theta" in bad.stderr and "vocab_size" in bad.stderr
    assert "Traceback" not in bad.stderr
    none = subprocess.run([sys.executable, "-m", "llmgen_b200", "info"], env={k: v for k, v in env.items() if k != "LLMGEN_MODEL"},
                          capture_output=True, text=True, timeout=300)
    assert none.returncode != 0 and "info needs --model" in none.stderr
