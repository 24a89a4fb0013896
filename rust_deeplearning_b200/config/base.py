"""Typed configuration helpers and the architecture registry.

The reference dispatches on a string in config.json
(`rustml/nlp/main/src/api/types.rs:521-524`) and silently falls back to GPT-2
for unknown names (`:743-779`).  Here one registry maps the architecture's name
to everything the library needs to know about it, and an unknown name is an
error that lists what is registered.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict


class ConfigError(ValueError):
    """A config.json that cannot describe a model: missing, ill-typed or inconsistent keys."""


_MISSING = object()


class ConfigReader:
    """Reads typed keys from a config.json dictionary and collects every problem before raising."""

    def __init__(self, raw: Dict[str, Any], what: str):
        if not isinstance(raw, dict):
            raise ConfigError(f"{what}: config.json must hold a JSON object")
        self.raw = raw
        self.what = what
        self.problems = []

    def _get(self, key, default):
        if key in self.raw and self.raw[key] is not None:
            return self.raw[key]
        if default is _MISSING:
            self.problems.append(f"missing key '{key}'")
            return None
        return default

    def integer(self, key, default=_MISSING, minimum=None, maximum=2 ** 31 - 1):
        """A whole number; by default at most 2^31 - 1, which is what the kernels' 32-bit indices hold."""
        v = self._get(key, default)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v.is_integer():
                v = int(v)
            else:
                self.problems.append(f"key '{key}' must be an integer, got {v!r}")
                return None
        if minimum is not None and v < minimum:
            self.problems.append(f"key '{key}' must be >= {minimum}, got {v}")
        if maximum is not None and v > maximum:
            self.problems.append(f"key '{key}' must be <= {maximum}, got {v}")
            return None
        return v

    def number(self, key, default=_MISSING, positive=False):
        v = self._get(key, default)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            self.problems.append(f"key '{key}' must be a number, got {v!r}")
            return None
        if not math.isfinite(v):
            self.problems.append(f"key '{key}' must be a finite number, got {v!r}")
            return None
        if positive and not v > 0:
            self.problems.append(f"key '{key}' must be > 0, got {v}")
        return float(v)

    def boolean(self, key, default=_MISSING):
        v = self._get(key, default)
        if v is None:
            return None
        if not isinstance(v, bool):
            self.problems.append(f"key '{key}' must be true or false, got {v!r}")
            return None
        return v

    def string(self, key, default=_MISSING):
        v = self._get(key, default)
        if v is None:
            return None
        if not isinstance(v, str):
            self.problems.append(f"key '{key}' must be a string, got {v!r}")
            return None
        return v

    def id_list(self, key, default=_MISSING):
        """An integer or a list of integers (eos_token_id is written both ways)."""
        v = self._get(key, default)
        if v is None:
            return None
        items = v if isinstance(v, (list, tuple)) else [v]
        out = []
        for item in items:
            if isinstance(item, bool) or not isinstance(item, int):
                self.problems.append(f"key '{key}' must be an integer or a list of integers, got {v!r}")
                return None
            out.append(item)
        return tuple(out)

    def check(self, ok: bool, message: str):
        if not ok:
            self.problems.append(message)

    def finish(self):
        if self.problems:
            raise ConfigError(f"{self.what}: " + "; ".join(self.problems))


@dataclass(frozen=True)
class Architecture:
    """What the library knows about one architecture: nothing else names it."""
    name: str                                   # config.json "architectures"[0]
    model_type: str                             # config.json "model_type"
    parse_config: Callable[[Dict[str, Any]], Any]   # dict -> typed configuration
    build_spec: Callable[[Any], Any]                # typed configuration -> parts.spec.ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture, replace: bool = False) -> None:
    if arch.name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture '{arch.name}' is already registered")
    _ARCHITECTURES[arch.name] = arch


def registered_architectures():
    return sorted(_ARCHITECTURES)


def architecture_for(raw: Dict[str, Any]) -> Architecture:
    """Choose by `architectures[0]`, else by `model_type`; an unknown name is an error."""
    if not isinstance(raw, dict):
        raise ConfigError("config.json must hold a JSON object")
    names = raw.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    if not isinstance(names, (list, tuple)):
        raise ConfigError(f"key 'architectures' must be a list of names, got {names!r}")
    for n in names:
        if isinstance(n, str) and n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    mt = raw.get("model_type")
    for arch in _ARCHITECTURES.values():
        if isinstance(mt, str) and arch.model_type == mt:
            return arch
    raise ConfigError(
        f"no registered architecture for architectures={names!r}, model_type={mt!r}; "
        f"registered: {registered_architectures()}")


def read_config_json(folder: str) -> Dict[str, Any]:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{folder}: no config.json in the model folder")
    with open(path) as f:
        try:
            return json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None


def load_config(folder_or_dict) -> Any:
    """Model folder (or an already parsed dictionary) -> the architecture's typed configuration."""
    raw = folder_or_dict if isinstance(folder_or_dict, dict) else read_config_json(folder_or_dict)
    return architecture_for(raw).parse_config(raw)
