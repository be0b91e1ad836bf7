"""One registry from an architecture's name (config.json ``architectures[0]``) to its model.

The reference has no registry: it hard-checks ``model_type == "qwen2"``
(src/flexengine/inference/models/qwen2.py:26).  An architecture here is a pair
(config class, plan builder); the plan builder turns the typed config into a
:class:`flexengine_b200.parts.spec.ModelPlan`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Mapping

from .model_config import ConfigError, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    build_plan: Callable


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, build_plan: Callable) -> None:
    """Make an architecture known.  ``config_class.from_dict(dict)`` must build the typed
    config; ``build_plan(config)`` must return a ModelPlan."""
    _ARCHITECTURES[name] = Architecture(name, config_class, build_plan)


def known_architectures() -> list[str]:
    _load_builtin()
    return sorted(_ARCHITECTURES)


def _load_builtin() -> None:
    # The built-in architecture registers itself on import.
    from .. import models  # noqa: F401


def architecture_of(config: Mapping) -> Architecture:
    _load_builtin()
    archs = config.get("architectures")
    if not archs or not isinstance(archs, (list, tuple)):
        raise ConfigError("config.json: key 'architectures' is missing or empty; known architectures: "
                          + ", ".join(sorted(_ARCHITECTURES)))
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(f"unknown architecture {name!r}; known architectures: " + ", ".join(sorted(_ARCHITECTURES)))
    return _ARCHITECTURES[name]


def resolve(config: Mapping):
    """config.json contents -> (typed config, ModelPlan)."""
    arch = architecture_of(config)
    typed = arch.config_class.from_dict(config)
    plan = arch.build_plan(typed)
    plan.validate()
    return typed, plan


def resolve_model_dir(model_dir: str):
    return resolve(read_config_json(model_dir))
