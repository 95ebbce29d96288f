"""What a model folder holds, without a GPU: the architecture's sizes, its tensors checked
against what the model declares, and what a prompt and a decode step cost.

The reference prints one line per model at start-up (`printInfo`, src/models/qwen3.zig:406-419:
layers, width, heads, head size, feed-forward width, vocabulary, eps, rotary base) and derives
FLOPs and bytes from the same sizes (src/profiler/metrics.zig:202-249); `describe` gives both,
layer by layer where layers differ, and `python -m llmgen_b200 info --model DIR` prints it.
"""
from __future__ import annotations

import math
import os
from collections import Counter
from typing import List, Optional

from .engine.profiler import ModelCost
from .parts.registry import model_weight_decls
from .parts.spec import MATRIX
from .registry import config_from_dict, config_from_folder


def _size(n_bytes: float) -> str:
    for unit, scale in (("GiB", 2 ** 30), ("MiB", 2 ** 20), ("KiB", 2 ** 10)):
        if n_bytes >= scale:
            return f"{n_bytes / scale:.2f} {unit}"
    return f"{int(n_bytes)} B"


def _layer_body(spec, item) -> str:
    block = spec.layers[item.layer]
    mixer, ffn = getattr(block, "mixer", None), getattr(block, "ffn", None)
    parts = []
    if getattr(mixer, "kind", None) == "attention":
        reach = f"window {mixer.window}" if mixer.window else "all keys"
        parts.append(f"attention {mixer.num_heads}/{mixer.num_kv_heads} heads x {mixer.head_dim}, {reach}")
    elif mixer is not None:
        parts.append(f"mixer '{getattr(mixer, 'kind', '?')}'")
    if getattr(ffn, "kind", None) == "gated_mlp":
        parts.append(f"gated feed-forward {ffn.intermediate_size} ({ffn.activation})")
    elif ffn is not None:
        parts.append(f"feed-forward '{getattr(ffn, 'kind', '?')}'")
    if item.cache is None:
        parts.append("no cache")
    elif not item.writes_cache:
        parts.append(f"reads cache {item.cache}")
    else:
        parts.append("a cache of its own")
    return ", ".join(parts)


def _run_list_lines(spec) -> List[str]:
    """The run list, consecutive items of the same make on one line."""
    lines, start = [], 0
    items = list(spec.run_order)
    bodies = [_layer_body(spec, item) for item in items]
    for i in range(1, len(items) + 1):
        if i == len(items) or bodies[i] != bodies[start]:
            layers = [it.layer for it in items[start:i]]
            name = f"layer {layers[0]}" if len(layers) == 1 else f"layers {layers[0]}-{layers[-1]}" \
                if layers == list(range(layers[0], layers[0] + len(layers))) else "layers " + ",".join(map(str, layers))
            lines.append(f"  {name}: {bodies[start]}")
            start = i
    return lines


def describe(model_dir: Optional[str] = None, config: Optional[dict] = None, context: int = 4096,
             check_tensors: bool = True) -> str:
    """Text about the model of a folder (config.json, and model.safetensors if it is there) or of a
    configuration dict.  Raises what the configuration reader or the weight loader raise: one error
    that lists every problem."""
    if (model_dir is None) == (config is None):
        raise ValueError("describe: give a model folder or a configuration, not both")
    arch, cfg = config_from_folder(model_dir) if model_dir is not None else config_from_dict(config)
    spec = arch.build_spec(cfg)
    decls = model_weight_decls(spec)
    n_all = sum(math.prod(d.shape) for d in decls)
    n_matrix = sum(math.prod(d.shape) for d in decls if d.kind == MATRIX)
    cost = ModelCost.from_spec(spec, w_elem=2, kv_elem=2)
    lines: List[str] = []
    first = spec.layers[spec.run_order[0].layer] if spec.run_order else None
    mixer, ffn = getattr(first, "mixer", None), getattr(first, "ffn", None)
    head = f"{spec.architecture}: layers={len(spec.run_order)}, hidden={spec.hidden_size}"
    if getattr(mixer, "kind", None) == "attention":
        head += f", heads={mixer.num_heads}/{mixer.num_kv_heads}, head_dim={mixer.head_dim}"
        if mixer.q_norm is not None:
            head += f", eps={mixer.q_norm.eps:g}"
        if mixer.position is not None:
            head += f", rope={mixer.position.theta:g}"
    if getattr(ffn, "kind", None) == "gated_mlp":
        head += f", ffn={ffn.intermediate_size}"
    head += (f", vocab={spec.vocab_size}, positions={spec.max_positions}, "
             f"{'tied' if spec.tied else 'untied'} output projection")
    lines.append(head)
    lines += _run_list_lines(spec)
    lines.append(f"  tensors: {len(decls)} declared, {n_all:,} values ({n_matrix:,} in matrices: "
                 f"{_size(n_matrix * 2)} in bfloat16, {_size(n_matrix * 4)} in float32)")
    lines.append(f"  in matrix products per token: {cost.n_mm:,} weights"
                 + ("" if cost.complete else " (parts of unknown kind not counted)"))
    lines.append(f"  cache: {cost.kv_bytes_per_token():,} bytes per token in bfloat16 "
                 f"({_size(cost.kv_bytes_per_token() * context)} for {context:,} tokens; windows not deducted)")
    lines.append(f"  a prompt of 2,048 tokens: {cost.prefill_flops(2048) / 1e9:,.1f} GFLOP; a decode step at {context:,} keys: "
                 f"{_size(cost.decode_bytes(context, 1))} read, {cost.decode_flops(context, 1) / 1e9:,.3f} GFLOP")
    if model_dir is not None and check_tensors:
        has_file = any(name.endswith(".safetensors") for name in os.listdir(model_dir))
        if has_file:
            from .weights import open_weights
            store = open_weights(model_dir, decls, spec.ignorable_tensors, spec.same_as)
            stored = Counter(str(store.directory.entry(d.name).dtype) for d in decls)
            lines.append("  model file: every declared tensor is there with its shape ("
                         + ", ".join(f"{n} stored as {k}" for k, n in sorted(stored.items())) + ")")
        else:
            lines.append("  model file: none in the folder (config.json only)")
    return "\n".join(lines)
