"""Typed configuration: the description of a model that every other part reads.

Three levels, all plain data:

* an *architecture config* (for instance :class:`Gemma2Config`) is read from the
  keys of the architecture's own ``config.json``;
* it is turned into a :class:`ModelSpec`: one :class:`LayerSpec` per layer, each
  naming its mixer, feed-forward, norms and position encoding with their sizes
  and constants as parameters, plus the *schedule*, the list that says in which
  order layers run and whose cache each call reads;
* the parts are built from the spec (``trapetum_b200.parts``), so that no part
  has to know which model it is in.

The reference keeps eleven numbers in a positional binary header
(model/export_gemma.py:55-58, runtime/src/lib.rs:4568-4573); here every size and
constant comes from ``config.json`` by key and is validated with an error that
names the key.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, replace
from typing import Any, Dict, List, Optional, Sequence, Tuple


class ConfigError(ValueError):
    """A key of config.json is missing, of the wrong type or out of range."""


_MISSING = object()


def _get(d: Dict[str, Any], key: str, typ, default=_MISSING, *, nullable=False):
    """Read ``key`` from ``d`` with a type check; the error names the key."""
    if key not in d or (d[key] is None and not nullable and default is not _MISSING):
        if default is _MISSING:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return default
    v = d[key]
    if v is None:
        if nullable:
            return None
        raise ConfigError(f"config.json: key '{key}' must not be null")
    if typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: key '{key}' must be a number, got {v!r}")
        return float(v)
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v == int(v):
                return int(v)
            raise ConfigError(f"config.json: key '{key}' must be an integer, got {v!r}")
        return int(v)
    if typ is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"config.json: key '{key}' must be true or false, got {v!r}")
        return v
    if typ is str:
        if not isinstance(v, str):
            raise ConfigError(f"config.json: key '{key}' must be a string, got {v!r}")
        return v
    raise TypeError(typ)


def _id_list(d: Dict[str, Any], key: str) -> Tuple[int, ...]:
    """A token id given as a number or as a list of numbers (the reference's
    server accepts both forms for ``eos_token_id``: runtime/src/bin/serve.rs:88-101)."""
    v = d.get(key)
    if v is None:
        return ()
    if isinstance(v, int) and not isinstance(v, bool):
        return (v,)
    if isinstance(v, (list, tuple)) and all(isinstance(x, int) and not isinstance(x, bool) for x in v):
        return tuple(v)
    raise ConfigError(f"config.json: key '{key}' must be an integer or a list of integers, got {v!r}")


# ----------------------------------------------------------------------------
# The spec of a model, layer by layer
# ----------------------------------------------------------------------------

@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: the registered ``kind`` and its parameters."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)

    def __hash__(self):  # params is a dict; identity of a spec is its content
        return hash((self.kind, json.dumps(self.params, sort_keys=True, default=str)))


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the arrangement (``block``) and the parts it arranges.

    ``prefix`` is the tensor-name prefix of the layer in the weight file; the
    names below it are the parts' own business.
    """
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    prefix: str


@dataclass(frozen=True)
class ScheduleEntry:
    """One call of a layer.  ``layer`` indexes ``ModelSpec.layers`` (a layer may
    be named by several entries and then runs with the same weights each time).
    ``cache_of`` names the *entry* whose cache this call uses: itself by
    default (the call appends its own keys and values, or owns its own state),
    or an earlier entry, whose cache it then only reads."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    max_positions: int
    stop_ids: Tuple[int, ...] = ()

    def validate(self) -> None:
        for e, ent in enumerate(self.schedule):
            if not (0 <= ent.layer < len(self.layers)):
                raise ConfigError(f"schedule entry {e} names layer {ent.layer}, "
                                  f"but the model has {len(self.layers)} layers")
            if ent.cache_of is not None:
                if not (0 <= ent.cache_of < e):
                    raise ConfigError(f"schedule entry {e} reads the cache of entry {ent.cache_of}, "
                                      f"which must be an earlier entry")
                if self.schedule[ent.cache_of].cache_of is not None:
                    raise ConfigError(f"schedule entry {e} reads the cache of entry {ent.cache_of}, "
                                      f"which does not own a cache itself")


def spec_to_json(spec: "ModelSpec") -> str:
    """The spec as JSON text, for the native host: part specs become ``{"kind", "params"}`` objects (also where
    they stand inside another part's parameters), tuples become lists."""
    def enc(v):
        if isinstance(v, PartSpec):
            return {"kind": v.kind, "params": {k: enc(x) for k, x in v.params.items()}}
        if isinstance(v, dict):
            return {str(k): enc(x) for k, x in v.items()}
        if isinstance(v, (list, tuple)):
            return [enc(x) for x in v]
        if isinstance(v, (str, int, float, bool)) or v is None:
            return v
        raise ConfigError(f"a spec value of type {type(v).__name__} cannot be handed to the native host: {v!r}")
    return json.dumps({
        "architecture": spec.architecture, "hidden_size": spec.hidden_size, "vocab_size": spec.vocab_size,
        "embedding": enc(spec.embedding), "final_norm": enc(spec.final_norm), "head": enc(spec.head),
        "layers": [{"prefix": l.prefix, "block": enc(l.block), "mixer": enc(l.mixer), "feed_forward": enc(l.feed_forward)}
                   for l in spec.layers],
        "schedule": [{"layer": e.layer, "cache_of": e.cache_of} for e in spec.schedule],
        "max_positions": spec.max_positions, "stop_ids": list(spec.stop_ids)})


# ----------------------------------------------------------------------------
# Registry: architecture name -> (config class, spec function)
# ----------------------------------------------------------------------------

_ARCHITECTURES: Dict[str, "ArchitectureEntry"] = {}


@dataclass(frozen=True)
class ArchitectureEntry:
    name: str
    config_cls: type
    to_spec: Any  # callable(config) -> ModelSpec


def register_architecture(name: str, config_cls: type, to_spec) -> None:
    """Make ``architectures[0] == name`` in a config.json select this model."""
    _ARCHITECTURES[name] = ArchitectureEntry(name, config_cls, to_spec)


def known_architectures() -> List[str]:
    return sorted(_ARCHITECTURES)


def architecture(name: str) -> ArchitectureEntry:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"unknown architecture '{name}'; known: {', '.join(known_architectures()) or '(none)'}") from None


def read_config_dict(path: str) -> Dict[str, Any]:
    """``path`` is a model folder or a config.json file."""
    p = os.path.join(path, "config.json") if os.path.isdir(path) else path
    try:
        with open(p, "r", encoding="utf-8") as f:
            d = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"no config.json at {p}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{p} is not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{p}: top level must be an object")
    return d


def architecture_name(d: Dict[str, Any]) -> str:
    archs = d.get("architectures")
    if not (isinstance(archs, list) and archs and isinstance(archs[0], str)):
        raise ConfigError("config.json: key 'architectures' must be a non-empty list of names")
    return archs[0]


def generation_stop_ids(folder: str) -> Tuple[int, ...]:
    """``eos_token_id`` (a number or a list) of the folder's generation_config.json, () if there is none.
    The reference's server reads this file before config.json and stops at the ids of both
    (runtime/src/bin/serve.rs:83-104)."""
    p = os.path.join(folder, "generation_config.json")
    if not os.path.isfile(p):
        return ()
    try:
        with open(p, "r", encoding="utf-8") as f:
            d = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{p} is not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{p}: top level must be an object")
    try:
        return _id_list(d, "eos_token_id")
    except ConfigError as e:
        raise ConfigError(str(e).replace("config.json", "generation_config.json")) from None


def load_config(path_or_dict) -> Tuple[Any, ModelSpec]:
    """Read a config.json and return (typed architecture config, ModelSpec).  For a model folder the stop
    ids are those of generation_config.json and of config.json together."""
    d = path_or_dict if isinstance(path_or_dict, dict) else read_config_dict(path_or_dict)
    entry = architecture(architecture_name(d))
    cfg = entry.config_cls.from_dict(d)
    spec = entry.to_spec(cfg)
    if not isinstance(path_or_dict, dict) and os.path.isdir(path_or_dict):
        more = generation_stop_ids(path_or_dict)
        if more:
            spec = replace(spec, stop_ids=tuple(sorted(set(more) | set(spec.stop_ids))))
    spec.validate()
    return cfg, spec
