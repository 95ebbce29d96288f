"""The reference's model file (GGUF) read and turned into a model folder (no GPU).  The files
are written here, by a writer of the test's own, in the layout the reference parses
(src/gguf.zig:361-480): header, typed metadata, tensor infos with the innermost dimension
first, data from the next multiple of the alignment."""
import json
import os
import struct
import subprocess
import sys

import pytest
import torch

from tests.util import ROOT, TINY_A, TINY_B

from llmgen_b200.engine.api import write_random_model
from llmgen_b200.parts.registry import model_weight_decls
from llmgen_b200.registry import config_from_dict
from llmgen_b200.weights import open_weights
from llmgen_b200.weights.gguf import GGUFError, GGUFFile, convert_gguf
from llmgen_b200.weights.safetensors_io import SafetensorsFile

U32, I32, F32, BOOL, STR, ARR, U64 = 4, 5, 6, 7, 8, 9, 10
TYPE_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 30}
THEIRS = {"input_layernorm": "attn_norm", "self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k",
          "self_attn.v_proj": "attn_v", "self_attn.o_proj": "attn_output", "self_attn.q_norm": "attn_q_norm",
          "self_attn.k_norm": "attn_k_norm", "post_attention_layernorm": "ffn_norm", "mlp.gate_proj": "ffn_gate",
          "mlp.up_proj": "ffn_up", "mlp.down_proj": "ffn_down"}


def gstr(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def gvalue(code, v) -> bytes:
    if code == STR:
        return gstr(v)
    if code == ARR:
        elem, items = v
        return struct.pack("<IQ", elem, len(items)) + b"".join(gvalue(elem, x) for x in items)
    return struct.pack({U32: "<I", I32: "<i", F32: "<f", BOOL: "<?", U64: "<Q"}[code], v)


def write_gguf(path, metadata, tensors, alignment=32, magic=0x46554747, type_codes=None):
    """metadata: [(key, type code, value)]; tensors: {name: torch tensor}."""
    head = struct.pack("<IIQQ", magic, 3, len(tensors), len(metadata))
    for key, code, v in metadata:
        head += gstr(key) + struct.pack("<I", code) + gvalue(code, v)
    blobs, offset = [], 0
    for name, t in tensors.items():
        raw = t.contiguous().view(torch.uint8).numpy().tobytes() if t.dtype != torch.bfloat16 \
            else t.contiguous().view(torch.int16).numpy().tobytes()
        code = (type_codes or {}).get(name, TYPE_CODE[t.dtype])
        head += gstr(name) + struct.pack("<I", t.dim()) + b"".join(struct.pack("<Q", d) for d in reversed(t.shape))
        head += struct.pack("<IQ", code, offset)
        pad = (-len(raw)) % alignment
        blobs.append(raw + b"\0" * pad)
        offset += len(raw) + pad
    head += b"\0" * ((-len(head)) % alignment)
    with open(path, "wb") as f:
        f.write(head + b"".join(blobs))


def their_name(ours: str) -> str:
    stem = ours[:-len(".weight")]
    if stem == "model.embed_tokens":
        return "token_embd.weight"
    if stem == "model.norm":
        return "output_norm.weight"
    if stem == "lm_head":
        return "output.weight"
    _, _, n, rest = stem.split(".", 3)
    return f"blk.{n}.{THEIRS[rest]}.weight"


def gguf_of(tmp_path, cfg, seed, rope_key="rope.freq_base", store=torch.bfloat16, drop=(), extra_meta=()):
    folder = write_random_model(str(tmp_path / f"src{seed}"), cfg, seed, store_dtype=store)
    stored = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {their_name(n): stored.tensor(n).clone() for n in stored.entries}
    meta = [("general.architecture", STR, "qwen3"), ("general.alignment", U32, 64),
            ("qwen3.block_count", U32, cfg["num_hidden_layers"]), ("qwen3.embedding_length", U32, cfg["hidden_size"]),
            ("qwen3.attention.head_count", U32, cfg["num_attention_heads"]),
            ("qwen3.attention.head_count_kv", U32, cfg["num_key_value_heads"]),
            ("qwen3.attention.key_length", U32, cfg["head_dim"]), ("qwen3.attention.value_length", U32, cfg["head_dim"]),
            ("qwen3.feed_forward_length", U64, cfg["intermediate_size"]),
            ("qwen3.context_length", U32, cfg["max_position_embeddings"]),
            ("qwen3.attention.layer_norm_rms_epsilon", F32, cfg["rms_norm_eps"]),
            (f"qwen3.{rope_key}", F32, cfg["rope_theta"]),
            ("tokenizer.ggml.tokens", ARR, (STR, [f"t{i}" for i in range(cfg["vocab_size"])])),
            ("tokenizer.ggml.eos_token_id", U32, 7), ("general.some_flag", BOOL, True)]
    meta = [m for m in meta if m[0] not in drop] + list(extra_meta)
    path = str(tmp_path / f"m{seed}.gguf")
    write_gguf(path, meta, tensors, alignment=64)
    return path, folder, tensors


@pytest.mark.parametrize("cfg,seed,store", [(TINY_A, 0, torch.bfloat16), (TINY_B, 1, torch.float32)])
def test_converted_folder_holds_the_same_model(tmp_path, cfg, seed, store):
    path, folder, tensors = gguf_of(tmp_path, cfg, seed, store=store)
    g = GGUFFile(path)
    assert g.version == 3 and g.architecture() == "qwen3" and g.metadata["general.some_flag"] is True
    assert g.tensors["blk.0.attn_q.weight"].shape == (cfg["num_attention_heads"] * cfg["head_dim"], cfg["hidden_size"])
    out = convert_gguf(path, str(tmp_path / "out"))
    got_cfg = json.load(open(os.path.join(out, "config.json")))
    for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                "num_key_value_heads", "head_dim", "rope_theta", "max_position_embeddings", "tie_word_embeddings"):
        assert got_cfg[key] == cfg[key], key
    assert abs(got_cfg["rms_norm_eps"] - cfg["rms_norm_eps"]) < 1e-12 and got_cfg["eos_token_id"] == 7
    # bit for bit the tensors of the folder the file was made from, under this engine's names
    a = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    b = SafetensorsFile(os.path.join(out, "model.safetensors"))
    assert sorted(a.entries) == sorted(b.entries)
    for name in a.entries:
        x, y = a.tensor(name), b.tensor(name)
        assert x.dtype == y.dtype and x.shape == y.shape and torch.equal(x.view(torch.uint8), y.view(torch.uint8)), name
    arch, typed = config_from_dict(got_cfg)
    open_weights(out, model_weight_decls(arch.build_spec(typed)))


def test_the_references_spelling_of_the_rotary_key_is_taken_and_none_is_refused(tmp_path):
    path, _, _ = gguf_of(tmp_path, TINY_A, 3, rope_key="rope.rope_freq_base")
    out = convert_gguf(path, str(tmp_path / "o"))
    assert json.load(open(os.path.join(out, "config.json")))["rope_theta"] == TINY_A["rope_theta"]
    path, _, _ = gguf_of(tmp_path, TINY_A, 4, drop=("qwen3.rope.freq_base", "qwen3.block_count"))
    with pytest.raises(GGUFError) as e:
        convert_gguf(path, str(tmp_path / "o2"))
    assert "qwen3.rope.freq_base or qwen3.rope.rope_freq_base" in str(e.value) and "qwen3.block_count" in str(e.value)


def test_files_that_cannot_be_read(tmp_path):
    t = {"token_embd.weight": torch.zeros(4, 8)}
    meta = [("general.architecture", STR, "qwen3")]
    bad = str(tmp_path / "bad.gguf")
    write_gguf(bad, meta, t, magic=0x12345678)
    with pytest.raises(GGUFError, match="bad magic"):
        GGUFFile(bad)
    write_gguf(bad, meta, t, type_codes={"token_embd.weight": 12})         # a quantized type
    with pytest.raises(GGUFError, match="ggml type 12"):
        GGUFFile(bad).tensor("token_embd.weight")
    write_gguf(bad, meta, t)
    with open(bad, "r+b") as f:
        f.truncate(os.path.getsize(bad) - 40)
    with pytest.raises(GGUFError, match="past the end"):
        GGUFFile(bad).tensor("token_embd.weight")
    with open(bad, "r+b") as f:
        f.truncate(30)
    with pytest.raises(GGUFError, match="ends inside its header"):
        GGUFFile(bad)
    write_gguf(bad, [("general.architecture", STR, "llama")], t)
    with pytest.raises(GGUFError, match="general.architecture is 'llama'"):
        convert_gguf(bad, str(tmp_path / "x"))
    path, _, tensors = gguf_of(tmp_path, TINY_A, 5)
    tensors["blk.0.attn_qq.weight"] = torch.zeros(2, 2)
    tensors["blk.9.attn_q.weight"] = torch.zeros(2, 2)
    g = GGUFFile(path)
    write_gguf(path, [(k, STR if isinstance(v, str) else (F32 if isinstance(v, float) else (BOOL if isinstance(v, bool) else
                      (ARR if isinstance(v, list) else U32))), (STR, v) if isinstance(v, list) else v)
                      for k, v in g.metadata.items()], tensors, alignment=64)
    with pytest.raises(GGUFError) as e:
        convert_gguf(path, str(tmp_path / "y"))
    assert "blk.0.attn_qq.weight" in str(e.value) and "blk.9.attn_q.weight" in str(e.value)


def test_convert_command(tmp_path):
    path, _, _ = gguf_of(tmp_path, TINY_B, 6, store=torch.float32)
    env = dict(os.environ, PYTHONPATH=ROOT)
    out = str(tmp_path / "folder")
    ok = subprocess.run([sys.executable, "-m", "llmgen_b200", "convert", path, out], env=env, capture_output=True,
                        text=True, timeout=300)
    assert ok.returncode == 0, ok.stderr
    assert "heads=8/1" in ok.stdout and "untied output projection" in ok.stdout
    assert "model file: every declared tensor is there" in ok.stdout and os.path.isfile(os.path.join(out, "model.safetensors"))
    bad = subprocess.run([sys.executable, "-m", "llmgen_b200", "convert", str(tmp_path / "none.gguf"), out], env=env,
                         capture_output=True, text=True, timeout=300)
    assert bad.returncode == 1 and "convert:" in bad.stderr and "Traceback" not in bad.stderr
    need = subprocess.run([sys.executable, "-m", "llmgen_b200", "convert", path], env=env, capture_output=True,
                          text=True, timeout=300)
    assert need.returncode != 0 and "convert needs the GGUF file and the folder" in need.stderr
