"""From the reference's model file to this engine's model folder.

The reference loads one GGUF file (src/gguf.zig:361-480): a header (magic "GGUF", version,
tensor count, metadata count), metadata as typed key/value pairs, tensor infos (name,
dimensions innermost first, type, offset) and, from the next multiple of `general.alignment`
(default 32), the tensor data.  This engine loads a folder with config.json and
model.safetensors.  `convert_gguf` reads the former and writes the latter:

  * sizes from the metadata keys the reference reads (src/models/qwen3.zig:100-140),
    `<arch>.block_count`, `.embedding_length`, `.attention.head_count[_kv]`,
    `.attention.key_length`, `.feed_forward_length`, `.context_length`,
    `.attention.layer_norm_rms_epsilon`, `<arch>.vocab_size` or the length of
    `tokenizer.ggml.tokens`, `tokenizer.ggml.eos_token_id`.  The rotary base is
    `<arch>.rope.freq_base`; the reference asks for `<arch>.rope.rope_freq_base` and silently
    falls back to 10000, here either spelling is taken and a file with neither is refused;
  * tensors by the reference's name table (src/models/qwen3.zig:34-55, src/module/trace.zig:47-59):
    `token_embd`, `output_norm`, `blk.N.attn_norm`, `attn_q/k/v`, `attn_output`, `attn_q_norm`,
    `attn_k_norm`, `ffn_norm`, `ffn_gate/up/down`, each with `.weight`; `output.weight`, where a
    file has it, becomes an untied `lm_head.weight` (the reference always ties).  Values are not
    touched: the rotary pairing of these files is the half-split one the engine uses, so no rows
    are permuted, and the reversed dimension order (src/gguf.zig:460) is only a relabelling;
  * types: 32-bit floats, 16-bit floats and bfloat16 (src/types.zig:18-37, the ones the reference
    uploads, src/memory/manager.zig:215-218); quantized types are refused by name.

Pure host code: `python -m llmgen_b200 convert model.gguf out_dir` needs no GPU.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from typing import Any, Dict, List, Tuple

import torch

GGUF_MAGIC = 0x46554747        # "GGUF", little endian
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_STRING, _ARRAY = 8, 9
_TENSOR_TYPES = {0: ("F32", torch.float32), 1: ("F16", torch.float16), 30: ("BF16", torch.bfloat16)}
MAX_DIMS = 4


class GGUFError(ValueError):
    pass


@dataclass(frozen=True)
class GGUFTensor:
    name: str
    shape: Tuple[int, ...]        # outermost first, as the engine names shapes
    type_code: int
    offset: int                   # from the start of the data section


class _Reader:
    def __init__(self, buf, path: str):
        self.buf, self.pos, self.path = buf, 0, path

    def take(self, fmt: str):
        size = struct.calcsize(fmt)
        if self.pos + size > len(self.buf):
            raise GGUFError(f"{self.path}: the file ends inside its header (at byte {self.pos})")
        (v,) = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += size
        return v

    def string(self) -> str:
        n = self.take("<Q")
        if self.pos + n > len(self.buf):
            raise GGUFError(f"{self.path}: a string of {n} bytes runs past the end of the file")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", "replace")
        self.pos += n
        return s

    def value(self, code: int, depth: int = 0) -> Any:
        if code in _SCALARS:
            return self.take(_SCALARS[code])
        if code == _STRING:
            return self.string()
        if code == _ARRAY and depth < 4:
            elem, count = self.take("<I"), self.take("<Q")
            if elem in _SCALARS and struct.calcsize(_SCALARS[elem]) * count > len(self.buf) - self.pos:
                raise GGUFError(f"{self.path}: an array of {count} values runs past the end of the file")
            return [self.value(elem, depth + 1) for _ in range(count)]
        raise GGUFError(f"{self.path}: unknown metadata type {code}")


class GGUFFile:
    """The metadata and the tensor table of a GGUF file; tensors are read on demand from a map of the file."""

    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as f:
            try:
                # a private copy-on-write map: torch wants a writable buffer, and nothing written reaches the file
                self._map = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY)
            except ValueError:
                raise GGUFError(f"{path}: the file is empty") from None
        r = _Reader(self._map, path)
        if r.take("<I") != GGUF_MAGIC:
            raise GGUFError(f"{path}: not a GGUF file (bad magic)")
        self.version = r.take("<I")
        n_tensors, n_meta = r.take("<Q"), r.take("<Q")
        self.metadata: Dict[str, Any] = {}
        for _ in range(n_meta):
            key = r.string()
            self.metadata[key] = r.value(r.take("<I"))
        self.tensors: Dict[str, GGUFTensor] = {}
        for _ in range(n_tensors):
            name = r.string()
            n_dims = r.take("<I")
            if n_dims > MAX_DIMS:
                raise GGUFError(f"{path}: tensor {name!r} has {n_dims} dimensions, at most {MAX_DIMS}")
            dims = [r.take("<Q") for _ in range(n_dims)]
            if any(d == 0 for d in dims):
                raise GGUFError(f"{path}: tensor {name!r} has an empty dimension")
            self.tensors[name] = GGUFTensor(name, tuple(reversed(dims)), r.take("<I"), r.take("<Q"))
        alignment = int(self.metadata.get("general.alignment", 32)) or 32
        self.data_start = (r.pos + alignment - 1) // alignment * alignment

    def architecture(self) -> str:
        return str(self.metadata.get("general.architecture", ""))

    def tensor(self, name: str) -> torch.Tensor:
        t = self.tensors.get(name)
        if t is None:
            raise GGUFError(f"{self.path}: no tensor {name!r}")
        if t.type_code not in _TENSOR_TYPES:
            raise GGUFError(f"{self.path}: tensor {name!r} has ggml type {t.type_code}; only F32 (0), F16 (1) and "
                            f"BF16 (30) are read, quantized files are not")
        _, dtype = _TENSOR_TYPES[t.type_code]
        n = 1
        for d in t.shape:
            n *= d
        begin = self.data_start + t.offset
        if begin + n * torch.empty((), dtype=dtype).element_size() > len(self._map):
            raise GGUFError(f"{self.path}: tensor {name!r} runs past the end of the file")
        return torch.frombuffer(self._map, dtype=dtype, count=n, offset=begin).reshape(t.shape).clone()


# the reference's names (left, `.weight` appended) and this engine's (right)
_GLOBAL_NAMES = {"token_embd": "model.embed_tokens", "output_norm": "model.norm"}
_LAYER_NAMES = {
    "attn_norm": "input_layernorm", "attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj",
    "attn_output": "self_attn.o_proj", "attn_q_norm": "self_attn.q_norm", "attn_k_norm": "self_attn.k_norm",
    "ffn_norm": "post_attention_layernorm", "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj",
}
ARCHITECTURES = {"qwen3": "Qwen3ForCausalLM"}


def config_from_metadata(g: GGUFFile) -> dict:
    """config.json of the model a GGUF file describes; one error lists every key that is missing."""
    arch = g.architecture()
    if arch not in ARCHITECTURES:
        raise GGUFError(f"{g.path}: general.architecture is {arch!r}; known: {', '.join(sorted(ARCHITECTURES))}")
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
        "architectures": [ARCHITECTURES[arch]], "model_type": arch,
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


def tensor_names(g: GGUFFile, num_layers: int) -> Dict[str, str]:
    """This engine's tensor name for every tensor of the file; unknown names are an error."""
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


def convert_gguf(path: str, out_dir: str) -> str:
    """Write config.json and model.safetensors for the model in the GGUF file `path`.  The folder is
    then checked the way every model folder is (missing, unexpected and misshapen tensors in one error)."""
    from ..parts.registry import model_weight_decls
    from ..registry import config_from_dict
    from .loader import open_weights
    from .random_init import write_model_folder
    g = GGUFFile(path)
    cfg = config_from_metadata(g)
    names = tensor_names(g, cfg["num_hidden_layers"])
    tensors = {ours: g.tensor(theirs) for theirs, ours in names.items()}
    arch, typed = config_from_dict(cfg, where=path)
    write_model_folder(out_dir, typed.to_dict() if hasattr(typed, "to_dict") else cfg, tensors,
                       metadata={"format": "pt", "converted_from": "gguf"})
    open_weights(out_dir, model_weight_decls(arch.build_spec(typed)))
    return out_dir
