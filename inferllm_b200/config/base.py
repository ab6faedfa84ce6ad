"""Architecture-neutral description of a decoder, and the base of typed configurations.

A configuration class (one per architecture) reads the architecture's own
`config.json` keys and turns them into a `ModelSpec`: a list of `LayerSpec`s (which
mixer, feed-forward, norm and block arrangement each layer has, with all sizes and
constants as parameters) and a schedule (the order in which layers run, as data).
Everything below the configuration (parts, cache, engine) sees only the `ModelSpec`.

The reference keeps the same split between a per-model class that reads the
hyper-parameters and builds the layer list (`LlamaLikeGraph::load_param` and
`construct_llm`, src/graph/llama_like.cpp:26-109) and generic modules that take their
sizes as constructor arguments (src/core/graph.h:84-205).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
    """A config.json that cannot be used: missing key, wrong type or unsupported value."""


@dataclass
class PartSpec:
    """Which implementation of a part (`kind`, a key of the part registries) and the
    sizes and constants it is built with."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)

    def __getitem__(self, key):
        return self.params[key]

    def get(self, key, default=None):
        return self.params.get(key, default)


@dataclass
class LayerSpec:
    """One layer: a block arrangement around a mixer and a feed-forward.

    `prefix` is the layer's tensor-name prefix in the weight file and `names` maps the
    block's roles ("mixer", "ffn", "norm1", "norm2", ...) to the sub-prefix below it;
    a part's own tensor names are appended to that."""

    block: str
    mixer: PartSpec
    ffn: PartSpec
    norm: PartSpec
    prefix: str
    names: Dict[str, str]


@dataclass
class ScheduleEntry:
    """One execution of a layer.  `layer` indexes `ModelSpec.layers` (a layer may be
    named by several entries: its weights are then used several times).  `cache` is the
    number of the cache entry that the mixer uses: entries with `writes=True` own it and
    append to it; an entry with `writes=False` only reads what an earlier entry of the
    same step wrote (a layer attending to another layer's keys and values)."""

    layer: int
    cache: int
    writes: bool = True


@dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    embedding: PartSpec          # params: name (tensor-name prefix)
    final_norm: PartSpec         # params: name, eps, ...
    head: PartSpec               # params: name, tied (bool)
    max_positions: int
    bos_token_id: Optional[int]
    eos_token_ids: List[int]

    def validate(self):
        seen_writer = {}
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ConfigError(f"schedule entry {i} names layer {e.layer}, "
                                  f"but there are {len(self.layers)} layers")
            if e.writes:
                if e.cache in seen_writer:
                    raise ConfigError(f"schedule entries {seen_writer[e.cache]} and {i} "
                                      f"both write cache entry {e.cache}")
                seen_writer[e.cache] = i
            elif e.cache not in seen_writer:
                raise ConfigError(f"schedule entry {i} reads cache entry {e.cache} "
                                  "before any entry has written it")


class ArchConfig:
    """Base of the typed configurations.  A subclass declares its fields as a dataclass,
    implements `from_dict` (the architecture's config.json keys -> fields, with
    validation), `to_dict` (back to those keys) and `model_spec`."""

    architecture: str = ""

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ArchConfig":
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:
        raise NotImplementedError

    def model_spec(self) -> ModelSpec:
        raise NotImplementedError


def read_config_json(folder: str) -> Dict[str, Any]:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{folder}: no config.json in this model folder")
    with open(path) as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return d


# ---- small typed readers used by the configuration classes


def take(d, key, typ, default=..., *, where="config.json"):
    """Read `d[key]` as `typ`; `default=...` makes the key required."""
    if key not in d or d[key] is None:
        if default is ...:
            raise ConfigError(f"{where}: required key '{key}' is missing")
        return default
    v = d[key]
    if typ is float and isinstance(v, int) and not isinstance(v, bool):
        v = float(v)
    if typ is int and isinstance(v, bool) or not isinstance(v, typ):
        raise ConfigError(f"{where}: key '{key}' must be {typ.__name__}, found {v!r}")
    return v
