"""Registries from a spec's `kind` to the class that runs it.

    register_mixer("attention", GQAAttention)       build_mixer(spec, ...)
    register_feed_forward("gated_mlp", GatedMLP)    build_feed_forward(spec, ...)
    register_norm("rmsnorm", RMSNorm)               build_norm(spec, ...)
    register_position("rope", Rope)                 build_position(spec, ...)
    register_block("prenorm", PreNormBlock)         build_block(spec, ...)

Every runtime class has `weight_decls(spec) -> [WeightDecl]` (a static method) and is
constructed as `cls(spec, weights, dtype, device)`; see `parts/base.py` for what else each
kind must offer.  A test or a user registers a new kind with one call; nothing else in the
framework names the kinds.
"""
from __future__ import annotations

from typing import Callable, Dict, List

from .spec import WeightDecl

_REGISTRIES: Dict[str, Dict[str, type]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {},
}


class PartError(ValueError):
    pass


def _register(family: str, kind: str, cls: type) -> type:
    _REGISTRIES[family][kind] = cls
    return cls


def _lookup(family: str, spec) -> type:
    _ensure_builtin()
    kind = getattr(spec, "kind", None)
    try:
        return _REGISTRIES[family][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRIES[family])) or "none"
        raise PartError(f"no {family} registered for kind {kind!r} (registered: {known})") from None


def register_mixer(kind: str, cls: type) -> type:
    return _register("mixer", kind, cls)


def register_feed_forward(kind: str, cls: type) -> type:
    return _register("feed_forward", kind, cls)


def register_norm(kind: str, cls: type) -> type:
    return _register("norm", kind, cls)


def register_position(kind: str, cls: type) -> type:
    return _register("position", kind, cls)


def register_block(kind: str, cls: type) -> type:
    return _register("block", kind, cls)


def mixer_class(spec) -> type:
    return _lookup("mixer", spec)


def feed_forward_class(spec) -> type:
    return _lookup("feed_forward", spec)


def norm_class(spec) -> type:
    return _lookup("norm", spec)


def position_class(spec) -> type:
    return _lookup("position", spec)


def block_class(spec) -> type:
    return _lookup("block", spec)


def build_mixer(spec, weights, dtype, device):
    return mixer_class(spec)(spec, weights, dtype, device)


def build_feed_forward(spec, weights, dtype, device):
    return feed_forward_class(spec)(spec, weights, dtype, device)


def build_norm(spec, weights, dtype, device):
    return norm_class(spec)(spec, weights, dtype, device)


def build_position(spec, weights, dtype, device):
    return position_class(spec)(spec, weights, dtype, device)


def build_block(spec, weights, dtype, device):
    return block_class(spec)(spec, weights, dtype, device)


def model_weight_decls(model_spec) -> List[WeightDecl]:
    """Every tensor a whole model reads, in declaration order."""
    _ensure_builtin()
    decls = [WeightDecl(model_spec.embedding, (model_spec.vocab_size, model_spec.hidden_size))]
    for layer in model_spec.layers:
        decls += block_class(layer).weight_decls(layer)
    decls += norm_class(model_spec.final_norm).weight_decls(model_spec.final_norm)
    if not model_spec.tied:
        decls.append(WeightDecl(model_spec.lm_head, (model_spec.vocab_size, model_spec.hidden_size)))
    return decls


def model_kernel_modules(model_spec) -> List[str]:
    """Names of the CUDA modules a model's parts launch (what its first call compiles)."""
    _ensure_builtin()
    mods = ["elementwise", "gemm_simt", "gemv", "gemm_tc", "sampling"]
    for layer in model_spec.layers:
        mods += list(block_class(layer).kernel_modules(layer))
    return list(dict.fromkeys(mods))


_builtin_loaded = False


def _ensure_builtin() -> None:
    global _builtin_loaded
    if not _builtin_loaded:
        _builtin_loaded = True
        from . import attention, block, mlp, norm, rope  # noqa: F401
