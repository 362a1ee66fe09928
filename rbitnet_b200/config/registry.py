"""One registry from an architecture's name to its configuration class and its model builder.

``config.json``'s ``architectures[0]`` chooses the entry, everywhere in the
package (engine, command line, trace replay).  The reference reads the
architecture name only for display (crates/bitnet-core/src/gguf/parse.rs:222-234)
and has a single model; here the name is the dispatch key so that a second
architecture is one ``register_architecture`` call.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Type

from .base import ModelConfig, ConfigError, read_config_json


@dataclass
class Architecture:
    name: str
    config_cls: Type[ModelConfig]
    #: config -> rbitnet_b200.parts.ModelSpec (layers, order, tensor names)
    build_spec: Callable


_REGISTRY: Dict[str, Architecture] = {}


def register_architecture(name: str, config_cls, build_spec, replace: bool = False) -> None:
    if name in _REGISTRY and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    _REGISTRY[name] = Architecture(name, config_cls, build_spec)


def unregister_architecture(name: str) -> None:
    _REGISTRY.pop(name, None)


def known_architectures():
    return sorted(_REGISTRY)


def get_architecture(name: str) -> Architecture:
    if name not in _REGISTRY:
        raise ConfigError(f"unknown architecture {name!r}; known: {', '.join(known_architectures())}")
    return _REGISTRY[name]


def architecture_of(config_dict) -> Architecture:
    archs = config_dict.get("architectures")
    if not archs or not isinstance(archs, list):
        raise ConfigError("config.json: missing architectures")
    return get_architecture(archs[0])


def config_from_dict(config_dict) -> ModelConfig:
    return architecture_of(config_dict).config_cls.from_dict(config_dict)


def load_config(folder) -> ModelConfig:
    return config_from_dict(read_config_json(folder))
