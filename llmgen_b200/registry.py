"""One registry from an architecture's name to its configuration class and its builder.

The reference's `ModelFactory` maps GGUF `general.architecture` to a creator and fails
with `error.UnknownArch` otherwise (src/models/factory.zig:46-72).  Here the key is
`config.json: architectures[0]` (or `model_type`), and an entry holds

    config_cls   typed configuration with `from_dict(dict, where) -> config`
    build_spec   function config -> `ModelSpec` (the model as data)

Adding an architecture is one `register_architecture` call; the engine, the cache manager,
trace replay and the command line find it through `resolve`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Iterable

from .config.base import ConfigError, architecture_name, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: type
    build_spec: Callable
    aliases: tuple = ()


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: type, build_spec: Callable,
                          aliases: Iterable[str] = ()) -> Architecture:
    arch = Architecture(name, config_cls, build_spec, tuple(aliases))
    for key in (name, *arch.aliases):
        _ARCHITECTURES[key] = arch
    return arch


def unregister_architecture(name: str) -> None:
    arch = _ARCHITECTURES.pop(name, None)
    if arch is not None:
        for key in arch.aliases:
            _ARCHITECTURES.pop(key, None)


def known_architectures() -> list:
    return sorted({a.name for a in _ARCHITECTURES.values()})


def resolve(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"unknown architecture {name!r}; registered: {', '.join(known_architectures())}") from None


def config_from_dict(data: dict, where: str = "config.json"):
    """(architecture entry, typed config) of a parsed config.json."""
    arch = resolve(architecture_name(data, where))
    return arch, arch.config_cls.from_dict(data, where)


def config_from_folder(model_dir: str):
    data = read_config_json(model_dir)
    return config_from_dict(data, where=f"{model_dir}/config.json")


_builtin_loaded = False


def _ensure_builtin() -> None:
    global _builtin_loaded
    if not _builtin_loaded:
        _builtin_loaded = True
        from . import models  # noqa: F401  (registers the built-in architectures)
