"""Random-weights mode: draw every declared tensor from a seed and write a model folder.

The reference has no such mode; it exists here so that tests and benchmarks need no
checkpoint.  Matrices and embedding tables are N(0, sigma); norm gains (the per-head q/k
norms too) are 1 + N(0, sigma_norm).  Each tensor has a generator of its own, seeded from
the run's seed and the tensor's name, so a tensor's values do not depend on which other
tensors exist or on the order of drawing.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterable

import torch

from ..parts.spec import INIT_ONE_PLUS_NORMAL, INT_TABLE, WeightDecl
from .loader import check_declarations
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensors(decls: Iterable[WeightDecl], seed: int, sigma: float, sigma_norm: float,
                   dtype: torch.dtype = torch.bfloat16, device="cpu") -> Dict[str, torch.Tensor]:
    """`device`: where the tensors are drawn and left.  The host's generator and a GPU's give different values
    for the same seed: model folders (and everything compared with the plain implementation) are drawn on the
    host; drawing on the GPU is for benchmarks of sizes whose tens of gigabytes would take minutes on the host."""
    out: Dict[str, torch.Tensor] = {}
    for name, d in check_declarations(list(decls)).items():
        g = torch.Generator(device=device)
        g.manual_seed(_tensor_seed(seed, name))
        if d.kind == INT_TABLE:
            out[name] = torch.randint(0, 2 ** 15, tuple(d.shape), generator=g, dtype=torch.int32, device=device)
            continue
        t = torch.empty(tuple(d.shape), dtype=torch.float32, device=device)
        if d.init == INIT_ONE_PLUS_NORMAL:
            t.normal_(0.0, sigma_norm, generator=g).add_(1.0)
        else:
            t.normal_(0.0, sigma, generator=g)
        out[name] = t.to(dtype)
    return out


def write_model_folder(model_dir: str, config_dict: dict, tensors: Dict[str, torch.Tensor],
                       metadata: Dict[str, str] | None = None) -> str:
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config_dict, f, indent=2)
        f.write("\n")
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors, metadata or {"format": "pt"})
    return model_dir
