"""The one registry: architecture name -> (config class, model builder).

The reference has a single model class and no registry (serve/api.py:52-64
rebuilds ``Transformer(ModelConfig(**cfg))`` directly).  Here config.json's
``architecture`` key picks an entry; the entry's config class parses the rest
of config.json and its builder turns that typed config into a model made of
parts.  Another architecture is another ``register_architecture`` call; no
framework file changes.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .model_config import ConfigError, read_config_json


@dataclass(frozen=True)
class ArchitectureEntry:
    name: str
    config_class: type          # has from_dict(dict) and to_dict()
    builder: Callable           # builder(config) -> parts.model.ComposedModel


_REGISTRY: dict[str, ArchitectureEntry] = {}
_NAME_ALIASES: dict[str, str] = {}


def register_architecture(name: str, config_class: type, builder: Callable,
                          aliases: tuple = ()) -> None:
    """Make ``name`` buildable.  ``builder(config)`` returns an unloaded model."""
    _REGISTRY[name] = ArchitectureEntry(name, config_class, builder)
    for a in aliases:
        _NAME_ALIASES[a] = name


def unregister_architecture(name: str) -> None:
    _REGISTRY.pop(name, None)
    for a in [a for a, n in _NAME_ALIASES.items() if n == name]:
        del _NAME_ALIASES[a]


def architecture_names() -> list:
    return sorted(_REGISTRY)


def lookup_architecture(name: str) -> ArchitectureEntry:
    _ensure_builtin()
    name = _NAME_ALIASES.get(name, name)
    if name not in _REGISTRY:
        raise ConfigError(
            f"unknown architecture {name!r}; registered: {architecture_names()}")
    return _REGISTRY[name]


def architecture_of(raw: dict) -> str:
    if "architecture" in raw:
        return raw["architecture"]
    archs = raw.get("architectures")
    if isinstance(archs, list) and archs:
        return archs[0]
    raise ConfigError("config.json names no architecture "
                      "(key 'architecture')")


def config_from_dict(raw: dict):
    """Typed config for a raw config.json dict, chosen by its architecture."""
    entry = lookup_architecture(architecture_of(raw))
    return entry.config_class.from_dict(raw)


def config_from_folder(folder):
    return config_from_dict(read_config_json(folder))


def build_model(config):
    """An unloaded model (parts with sizes, no weights) for a typed config."""
    return lookup_architecture(config.architecture).builder(config)


_builtin_done = False


def _ensure_builtin() -> None:
    global _builtin_done
    if not _builtin_done:
        _builtin_done = True
        from ..parts import llama_dense  # noqa: F401  (registers itself)
