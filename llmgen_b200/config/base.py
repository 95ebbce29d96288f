"""Helpers for typed model configurations read from a model folder's config.json.

A configuration class is a frozen dataclass whose fields are the architecture's own
config.json keys.  `ConfigReader` pulls keys out of the parsed JSON, records every
problem it meets (missing key, wrong type, value out of range) and raises them all
at once as one `ConfigError`, so a user sees the whole list and not the first item.

The reference reads its typed `Config` from GGUF metadata with silent defaults of 0
(src/models/qwen3.zig:97-139); here a key that the model needs and the file does not
give is an error, never a constant in code.
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Sequence


class ConfigError(ValueError):
    """Raised for a config.json that cannot describe a runnable model."""


_MISSING = object()


class ConfigReader:
    """Collects typed values from a config dict and the problems met on the way."""

    def __init__(self, data: dict, where: str = "config.json"):
        if not isinstance(data, dict):
            raise ConfigError(f"{where}: top level must be a JSON object")
        self.data = data
        self.where = where
        self.problems: list[str] = []

    # -- typed getters -------------------------------------------------
    def _get(self, key: str, default: Any = _MISSING) -> Any:
        if key in self.data and self.data[key] is not None:
            return self.data[key]
        if default is _MISSING:
            self.problems.append(f"missing key '{key}'")
            return None
        return default

    def integer(self, key: str, default: Any = _MISSING, minimum: int | None = 1) -> int | None:
        v = self._get(key, default)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v == int(v):
                v = int(v)
            else:
                self.problems.append(f"'{key}' must be an integer, got {v!r}")
                return None
        if minimum is not None and v < minimum:
            self.problems.append(f"'{key}' must be >= {minimum}, got {v}")
            return None
        return v

    def number(self, key: str, default: Any = _MISSING, positive: bool = True) -> float | None:
        v = self._get(key, default)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            self.problems.append(f"'{key}' must be a number, got {v!r}")
            return None
        if positive and not v > 0:
            self.problems.append(f"'{key}' must be > 0, got {v}")
            return None
        return float(v)

    def boolean(self, key: str, default: Any = _MISSING) -> bool | None:
        v = self._get(key, default)
        if v is None:
            return None
        if not isinstance(v, bool):
            self.problems.append(f"'{key}' must be true or false, got {v!r}")
            return None
        return v

    def string(self, key: str, default: Any = _MISSING, choices: Sequence[str] | None = None) -> str | None:
        v = self._get(key, default)
        if v is None:
            return None
        if not isinstance(v, str):
            self.problems.append(f"'{key}' must be a string, got {v!r}")
            return None
        if choices is not None and v not in choices:
            self.problems.append(f"'{key}' = {v!r} is not supported (supported: {', '.join(choices)})")
            return None
        return v

    def raw(self, key: str, default: Any = None) -> Any:
        return self.data.get(key, default)

    def problem(self, text: str) -> None:
        self.problems.append(text)

    def check(self, ok: bool, text: str) -> None:
        if not ok:
            self.problems.append(text)

    def finish(self) -> None:
        if self.problems:
            raise ConfigError(f"{self.where}: " + "; ".join(self.problems))


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no such file (a model folder holds config.json and model.safetensors)")
    with open(path, "r", encoding="utf-8") as f:
        try:
            data = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(data, dict):
        raise ConfigError(f"{path}: top level must be a JSON object")
    return data


def architecture_name(data: dict, where: str = "config.json") -> str:
    """The registry key of a config dict: `architectures[0]`, else `model_type`.

    The reference keys its registry by GGUF `general.architecture`
    (src/models/factory.zig:68-71); for a config.json folder the same role is played by
    the `architectures` list.
    """
    archs = data.get("architectures")
    if isinstance(archs, list) and archs and isinstance(archs[0], str):
        return archs[0]
    mt = data.get("model_type")
    if isinstance(mt, str) and mt:
        return mt
    raise ConfigError(f"{where}: neither 'architectures' nor 'model_type' names the model")
