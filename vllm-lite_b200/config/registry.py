"""One registry from an architecture's name to its configuration class and to
the function that turns a configuration into a `ModelPlan`.

The name is `architectures[0]` of config.json.  When that key is absent the
reference's rule applies: `model_type`, lower-cased, among the names an entry
claims (crates/model/src/qwen3/arch.rs:40-50; the reference's registry is a map
name -> factory behind a lock, crates/model/src/arch/registry.rs:98-113)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Tuple

from .errors import ConfigError, UnknownArchitecture


@dataclass(frozen=True)
class ArchitectureEntry:
    name: str
    config_cls: type
    plan: Callable                      # config -> ModelPlan
    model_types: Tuple[str, ...] = ()


_REGISTRY = {}


def register_architecture(name, config_cls, plan, model_types=(), replace=False):
    if name in _REGISTRY and not replace:
        raise KeyError(f"architecture {name!r} is already registered")
    _REGISTRY[name] = ArchitectureEntry(name, config_cls, plan, tuple(m.lower() for m in model_types))
    return _REGISTRY[name]


def unregister_architecture(name):
    _REGISTRY.pop(name, None)


def registered_architectures():
    return sorted(_REGISTRY)


def resolve_architecture(config_json: dict) -> ArchitectureEntry:
    if not isinstance(config_json, dict):
        raise ConfigError("config.json must hold a JSON object")
    archs = config_json.get("architectures")
    if isinstance(archs, list) and archs:
        name = archs[0]
        if name in _REGISTRY:
            return _REGISTRY[name]
        raise UnknownArchitecture(name, _REGISTRY)
    model_type = str(config_json.get("model_type", "")).lower()
    for entry in _REGISTRY.values():
        if model_type and model_type in entry.model_types:
            return entry
    raise UnknownArchitecture(model_type or "(no `architectures`, no `model_type`)", _REGISTRY)


def plan_from_config_json(config_json: dict):
    """(typed configuration, ModelPlan) for a parsed config.json."""
    entry = resolve_architecture(config_json)
    cfg = entry.config_cls.from_dict(config_json)
    return cfg, entry.plan(cfg).validate()
