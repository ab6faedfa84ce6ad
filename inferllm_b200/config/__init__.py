"""Configurations and the registry of architectures, as Python sees them.

The typed configurations, the registry and the architecture-neutral ModelSpec live in the C++ core
(`config/config.h`, `config/llama.h`); this module is their face.  `config_from_dict` /
`config_from_folder` return a configuration object whose attributes are the architecture's own
config.json keys; `model_spec()` gives the ModelSpec as data (`PartSpec`, `LayerSpec`,
`ScheduleEntry`).  An architecture can also be written in Python: subclass `ArchConfig`
(`from_dict`, `to_dict`, `model_spec`) and `register_architecture(name, cls)`; the library then
builds its generic decoder from the spec that the class returns.
"""
from __future__ import annotations

import ctypes
import json
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .. import binding as _b
from ..binding import ConfigError


@dataclass
class PartSpec:
    """Which implementation of a part (`kind`, a key of the part registries) and the sizes and
    constants it is built with.  A parameter may itself be a part (a PartSpec)."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)

    def __getitem__(self, key):
        return self.params[key]

    def get(self, key, default=None):
        return self.params.get(key, default)

    def to_json(self):
        return {"kind": self.kind, "params": {k: (v.to_json() if isinstance(v, PartSpec) else v)
                                              for k, v in self.params.items()}}

    @staticmethod
    def from_json(j):
        params = {k: (PartSpec.from_json(v) if isinstance(v, dict) and "kind" in v and "params" in v else v)
                  for k, v in j.get("params", {}).items()}
        return PartSpec(j["kind"], params)


@dataclass
class LayerSpec:
    """One layer: a block arrangement around a mixer and a feed-forward; `norms` gives each norm role
    of the block a spec of its own; `prefix` and `names` place the layer's tensors in the weight file."""

    block: str
    mixer: PartSpec
    ffn: PartSpec
    norms: Dict[str, PartSpec]
    prefix: str
    names: Dict[str, str]


@dataclass
class ScheduleEntry:
    """One execution of a layer: `layer` indexes ModelSpec.layers, `cache` numbers the cache entry the
    mixer uses, `writes=False` only reads what an earlier entry of the same step wrote."""

    layer: int
    cache: int
    writes: bool = True


@dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    embedding: PartSpec
    final_norm: PartSpec
    head: PartSpec
    max_positions: int
    bos_token_id: Optional[int]
    eos_token_ids: List[int]

    def to_json(self):
        return {"hidden_size": self.hidden_size, "vocab_size": self.vocab_size, "max_positions": self.max_positions,
                "bos_token_id": self.bos_token_id, "eos_token_ids": list(self.eos_token_ids),
                "embedding": self.embedding.to_json(), "final_norm": self.final_norm.to_json(), "head": self.head.to_json(),
                "layers": [{"block": ls.block, "mixer": ls.mixer.to_json(), "ffn": ls.ffn.to_json(),
                            "norms": {r: n.to_json() for r, n in ls.norms.items()}, "prefix": ls.prefix,
                            "names": dict(ls.names)} for ls in self.layers],
                "schedule": [{"layer": e.layer, "cache": e.cache, "writes": e.writes} for e in self.schedule]}

    @staticmethod
    def from_json(j):
        layers = [LayerSpec(ls["block"], PartSpec.from_json(ls["mixer"]), PartSpec.from_json(ls["ffn"]),
                            {r: PartSpec.from_json(n) for r, n in ls["norms"].items()}, ls["prefix"], dict(ls["names"]))
                  for ls in j["layers"]]
        return ModelSpec(j["hidden_size"], j["vocab_size"], layers,
                         [ScheduleEntry(e["layer"], e["cache"], e.get("writes", True)) for e in j["schedule"]],
                         PartSpec.from_json(j["embedding"]), PartSpec.from_json(j["final_norm"]), PartSpec.from_json(j["head"]),
                         j["max_positions"], j.get("bos_token_id"), list(j.get("eos_token_ids", [])))

    def validate(self):
        """ConfigError for a schedule that names no layer, writes an entry twice or reads before writing."""
        _b.check(_b.lib().illm_model_spec_validate(json.dumps(self.to_json()).encode()))


class _Handle:
    """Owns a configuration object of the library."""

    def __init__(self, ptr):
        self.ptr = ptr

    def __del__(self):
        if self.ptr and _b._lib is not None:
            _b._lib.illm_config_free(self.ptr)
            self.ptr = None


class ArchConfig:
    """Base of the typed configurations.  A configuration of an architecture that the library knows
    itself is a `LibraryConfig`; one written in Python subclasses this class directly, implements
    `from_dict`, `to_dict` and `model_spec`, and is registered with `register_architecture`."""

    architecture: str = ""
    _handle: Optional[_Handle] = None

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ArchConfig":
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:
        raise NotImplementedError

    def model_spec(self) -> ModelSpec:
        raise NotImplementedError

    def handle(self):
        """The library's object for this configuration (made on first use)."""
        if self._handle is None:
            out = ctypes.c_void_p()
            _b.check(_b.lib().illm_config_from_json(json.dumps(self.to_dict()).encode(), _b.enc(self.architecture),
                                                    ctypes.byref(out)))
            self._handle = _Handle(out)
        return self._handle.ptr


class LibraryConfig(ArchConfig):
    """A configuration of an architecture implemented in the library: the attributes are the keys of
    its `to_dict()` (the architecture's own config.json keys, defaults filled in)."""

    def __init__(self, handle: _Handle):
        self._handle = handle
        self._dict = _b.call_json(_b.lib().illm_config_to_json, handle.ptr)
        self.architecture = _b.call_text(_b.lib().illm_config_architecture, handle.ptr)

    def __getattr__(self, name):
        d = self.__dict__.get("_dict", {})
        if name in d:
            return d[name]
        raise AttributeError(name)

    def __eq__(self, other):
        return isinstance(other, LibraryConfig) and self._dict == other._dict

    def __repr__(self):
        return f"{type(self).__name__}({self._dict})"

    @classmethod
    def from_dict(cls, d):
        out = ctypes.c_void_p()
        _b.check(_b.lib().illm_config_from_json(json.dumps(d).encode(), _b.enc(cls.architecture) or None, ctypes.byref(out)))
        return cls(_Handle(out))

    def to_dict(self):
        return dict(self._dict)

    def model_spec(self):
        return ModelSpec.from_json(_b.call_json(_b.lib().illm_config_model_spec, self._handle.ptr))


class LlamaConfig(LibraryConfig):
    """The LLaMA dense decoder (`config/llama.h`): hidden_size, num_hidden_layers, num_attention_heads,
    num_key_value_heads, head_dim, intermediate_size, vocab_size, rms_norm_eps, rope_theta,
    max_position_embeddings, tie_word_embeddings, bos_token_id, eos_token_id (a list), torch_dtype."""

    architecture = "LlamaForCausalLM"

    def __getattr__(self, name):
        if name == "eos_token_id":
            e = self.__dict__.get("_dict", {}).get("eos_token_id")
            return list(e) if isinstance(e, list) else [e]
        return super().__getattr__(name)


_PY_CLASSES: Dict[str, type] = {"LlamaForCausalLM": LlamaConfig}
_CALLBACKS = {}      # name -> (ctypes callback, holder of the last returned text): kept alive while registered


def registered_architectures() -> List[str]:
    return _b.call_json(_b.lib().illm_registered_architectures)


def resolve_architecture(name: str) -> str:
    """The registered name behind a name or an alias; ConfigError listing what is registered otherwise."""
    return _b.call_text(_b.lib().illm_resolve_architecture, name.encode())


def config_class(name: str) -> type:
    return _PY_CLASSES.get(resolve_architecture(name), LibraryConfig)


def register_architecture(name: str, config_cls: type, aliases=()):
    """Register (or replace) an architecture written in Python: `config_cls.from_dict(d)` makes the
    typed configuration, its `to_dict()` and `model_spec()` describe it to the library, which builds
    the generic decoder from the spec."""
    holder = {}

    def describe(_user, config_json):
        try:
            cfg = config_cls.from_dict(json.loads(config_json.decode()))
            text = json.dumps({"config": cfg.to_dict(), "spec": cfg.model_spec().to_json()})
        except Exception as e:      # reported by the library as a ConfigError
            text = json.dumps({"error": f"{type(e).__name__}: {e}"})
        holder["text"] = ctypes.create_string_buffer(text.encode())      # stays valid until the next call
        return ctypes.addressof(holder["text"])

    cb = ctypes.CFUNCTYPE(ctypes.c_void_p, ctypes.c_void_p, ctypes.c_char_p)(describe)
    _b.check(_b.lib().illm_register_architecture(name.encode(), json.dumps(list(aliases)).encode(),
                                                 ctypes.cast(cb, ctypes.c_void_p), None))
    _CALLBACKS[name] = (cb, holder)
    _PY_CLASSES[name] = config_cls
    config_cls.architecture = name


def unregister_architecture(name: str):
    _b.check(_b.lib().illm_unregister_architecture(name.encode()))
    _CALLBACKS.pop(name, None)
    if _PY_CLASSES.get(name) is not LlamaConfig:
        _PY_CLASSES.pop(name, None)


def config_from_dict(d: dict, model_name: Optional[str] = None) -> ArchConfig:
    """Typed configuration of a config.json dictionary; the class is chosen by `architectures[0]`
    unless `model_name` overrides it."""
    out = ctypes.c_void_p()
    _b.check(_b.lib().illm_config_from_json(json.dumps(d).encode(), _b.enc(model_name), ctypes.byref(out)))
    handle = _Handle(out)
    arch = _b.call_text(_b.lib().illm_config_architecture, handle.ptr)
    cls = _PY_CLASSES.get(arch, LibraryConfig)
    if issubclass(cls, LibraryConfig):
        return cls(handle)
    cfg = cls.from_dict(d)
    cfg._handle = handle
    return cfg


def config_from_folder(folder: str, model_name: Optional[str] = None) -> ArchConfig:
    out = ctypes.c_void_p()
    _b.check(_b.lib().illm_config_from_folder(folder.encode(), _b.enc(model_name), ctypes.byref(out)))
    handle = _Handle(out)
    arch = _b.call_text(_b.lib().illm_config_architecture, handle.ptr)
    cls = _PY_CLASSES.get(arch, LibraryConfig)
    if issubclass(cls, LibraryConfig):
        return cls(handle)
    with open(f"{folder}/config.json") as f:
        cfg = cls.from_dict(json.load(f))
    cfg._handle = handle
    return cfg
