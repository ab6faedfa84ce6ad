"""The one registry from an architecture's name to its configuration class and model.

The reference maps a model name to a Graph subclass in an if-chain and aborts on an
unknown name (`Graph::make_graph`, src/graph/graph_imp.cpp:6-21).  Here the name is
`architectures[0]` of config.json (or one of the registered aliases, among them the
reference's own names "llama" and "llama2"), and an unknown name is an error that
lists what is registered.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional, Type

from .config.base import ArchConfig, ConfigError, read_config_json


@dataclass
class Architecture:
    name: str
    config_cls: Type[ArchConfig]
    build_model: Callable  # (config, runtime) -> model object (see models/decoder.py)


_ARCHITECTURES: Dict[str, Architecture] = {}
_ALIASES: Dict[str, str] = {}


def register_architecture(name: str, config_cls: Type[ArchConfig],
                          build_model: Optional[Callable] = None, aliases=()) -> Architecture:
    """Register (or replace) an architecture.  `build_model(config, runtime)` defaults to
    the generic decoder built from `config.model_spec()`."""
    if build_model is None:
        def build_model(config, runtime):
            from .models.decoder import DecoderModel
            return DecoderModel(config.model_spec(), runtime)
    arch = Architecture(name, config_cls, build_model)
    _ARCHITECTURES[name] = arch
    for a in aliases:
        _ALIASES[a] = name
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)
    for a in [a for a, n in _ALIASES.items() if n == name]:
        del _ALIASES[a]


def get_architecture(name: str) -> Architecture:
    key = _ALIASES.get(name, name)
    if key not in _ARCHITECTURES:
        known = sorted(_ARCHITECTURES) + sorted(_ALIASES)
        raise ConfigError(f"unknown architecture '{name}'; registered: {', '.join(known)}")
    return _ARCHITECTURES[key]


def registered_architectures():
    return sorted(_ARCHITECTURES)


def config_from_dict(d: dict, model_name: Optional[str] = None) -> ArchConfig:
    """Typed configuration of a config.json dictionary; the class is chosen by
    `architectures[0]` unless `model_name` overrides it."""
    if model_name is None:
        archs = d.get("architectures")
        if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
            raise ConfigError("config.json: required key 'architectures' (a list with the "
                              "model class name) is missing")
        model_name = archs[0]
    return get_architecture(model_name).config_cls.from_dict(d)


def config_from_folder(folder: str, model_name: Optional[str] = None) -> ArchConfig:
    return config_from_dict(read_config_json(folder), model_name)


def _register_builtin():
    from .config.llama import LlamaConfig
    register_architecture("LlamaForCausalLM", LlamaConfig, aliases=("llama", "llama2"))


_register_builtin()
