"""The one registry from an architecture's name (``architectures[0]`` of config.json) to its typed
configuration class and its spec builder.  The reference has none: it runs one pinned model
(ampere_kv/runner.py:13-14, docs/ARCHITECTURE.md:3)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

from ..config.model_config import ConfigError, read_config_json
from ..config.spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any
    build_spec: Callable[[Any], ModelSpec]


ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class, build_spec) -> Architecture:
    arch = Architecture(name, config_class, build_spec)
    ARCHITECTURES[name] = arch
    return arch


def architecture_of(raw_config: dict) -> Architecture:
    names = raw_config.get("architectures")
    if not names or not isinstance(names, (list, tuple)) or not isinstance(names[0], str):
        raise ConfigError("config.json: key 'architectures' must be a non-empty list of names")
    if names[0] not in ARCHITECTURES:
        raise ConfigError(f"config.json: architecture {names[0]!r} is not registered; known: {sorted(ARCHITECTURES)}")
    return ARCHITECTURES[names[0]]


def load_config(model_dir: str):
    """(architecture, typed config) of a model folder."""
    from . import qwen3  # noqa: F401  (registers the built-in architecture)
    raw = read_config_json(model_dir)
    arch = architecture_of(raw)
    return arch, arch.config_class.from_dict(raw)


def config_from_dict(raw: dict):
    from . import qwen3  # noqa: F401
    arch = architecture_of(raw)
    return arch, arch.config_class.from_dict(raw)
