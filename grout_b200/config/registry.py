"""One registry from an architecture's name to its configuration class and to
the function that lays the model out from that configuration.

The reference has no registry: it accepts ``model_type == "qwen3"`` and nothing
else (src/engine.rs:24-29).  Here config.json's ``architectures[0]`` chooses the
entry and ``model_type`` is the fallback, so that another architecture is one
``register_architecture`` call away and no caller names a model class.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Tuple

from .base import ConfigError, ModelConfig, read_json
import os


@dataclass(frozen=True)
class Architecture:
    name: str                                   # e.g. "Qwen3ForCausalLM"
    model_types: Tuple[str, ...]                # config.json "model_type" values
    config_cls: type
    plan: Callable[[ModelConfig], "object"]     # config -> parts.plan.ModelPlan


_BY_NAME: Dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: type, plan: Callable, model_types=()) -> Architecture:
    """Adds (or replaces) an architecture.  ``plan(config)`` returns the
    ``ModelPlan`` that the engine builds the model from."""
    arch = Architecture(name, tuple(model_types), config_cls, plan)
    _BY_NAME[name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _BY_NAME.pop(name, None)


def known_architectures():
    return sorted(_BY_NAME)


def resolve_architecture(raw: dict, where: str = "config.json") -> Architecture:
    names = raw.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    for n in names:
        if n in _BY_NAME:
            return _BY_NAME[n]
    mt = raw.get("model_type")
    if mt is not None:
        for arch in _BY_NAME.values():
            if mt in arch.model_types:
                return arch
    raise ConfigError([f"no registered architecture for architectures={list(names)!r}, "
                       f"model_type={mt!r}; known: {known_architectures()}"], where)


def load_config(model_dir: str):
    """Reads ``model_dir/config.json`` and returns (architecture, typed config)."""
    path = os.path.join(model_dir, "config.json")
    raw = read_json(path)
    arch = resolve_architecture(raw, path)
    return arch, arch.config_cls.from_dict(raw, path)
