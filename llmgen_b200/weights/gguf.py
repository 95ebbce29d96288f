"""From the reference's model file to this engine's model folder.

The reference loads one GGUF file (src/gguf.zig:361-480): a header (magic "GGUF", version,
tensor count, metadata count), metadata as typed key/value pairs, tensor infos (name,
dimensions innermost first, type, offset) and, from the next multiple of `general.alignment`
(default 32), the tensor data.  This engine loads a folder with config.json and
model.safetensors.  `convert_gguf` reads the former and writes the latter; what depends on the
architecture (metadata keys, tensor names) is registered by the architecture's module
(`register_gguf_source`; for Qwen3 in models/qwen3.py):

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
from typing import Any, Callable, Dict, Tuple

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


@dataclass(frozen=True)
class GGUFSource:
    """How one architecture's GGUF files become a model folder: `config(file) -> dict` (config.json keys) and
    `names(file, config) -> {name in the file: this engine's tensor name}`."""
    config: Callable[["GGUFFile"], dict]
    names: Callable[["GGUFFile", dict], Dict[str, str]]


_SOURCES: Dict[str, GGUFSource] = {}


def register_gguf_source(gguf_architecture: str, config: Callable, names: Callable) -> None:
    """`gguf_architecture` is the file's `general.architecture` (src/gguf.zig:224-226)."""
    _SOURCES[gguf_architecture] = GGUFSource(config, names)


def gguf_source(g: "GGUFFile") -> GGUFSource:
    from ..registry import _ensure_builtin
    _ensure_builtin()                          # the built-in architectures register their sources when they are loaded
    arch = g.architecture()
    if arch not in _SOURCES:
        raise GGUFError(f"{g.path}: general.architecture is {arch!r}; known: {', '.join(sorted(_SOURCES)) or 'none'}")
    return _SOURCES[arch]


def convert_gguf(path: str, out_dir: str) -> str:
    """Write config.json and model.safetensors for the model in the GGUF file `path`.  The folder is
    then checked the way every model folder is (missing, unexpected and misshapen tensors in one error)."""
    from ..parts.registry import model_weight_decls
    from ..registry import config_from_dict
    from .loader import open_weights
    from .random_init import write_model_folder
    g = GGUFFile(path)
    source = gguf_source(g)
    cfg = source.config(g)
    names = source.names(g, cfg)
    tensors = {ours: g.tensor(theirs) for theirs, ours in names.items()}
    arch, typed = config_from_dict(cfg, where=path)
    write_model_folder(out_dir, typed.to_dict() if hasattr(typed, "to_dict") else cfg, tensors,
                       metadata={"format": "pt", "converted_from": "gguf"})
    open_weights(out_dir, model_weight_decls(arch.build_spec(typed)))
    return out_dir
