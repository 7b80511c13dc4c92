"""One registry from an architecture's name to its configuration class and model plan.

The reference has none: its runner imports ``Qwen3ForCausalLM`` by name
(engine/model_runner.py:5,36).  Here ``config.json["architectures"][0]`` selects an
``Architecture`` everywhere (engine, trace replay, random weights), and a new one is
added by calling ``register_architecture`` — from a file of the package or from a
test — without touching the engine.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

from .model_config import ConfigError, ModelConfig, architecture_name, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable[[dict[str, Any]], ModelConfig]
    # config -> parts.model.ModelPlan (what layers exist, of which parts, run in which order)
    plan: Callable[[ModelConfig], Any]


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture, *, replace: bool = False) -> None:
    if arch.name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture {arch.name!r} is already registered")
    _ARCHITECTURES[arch.name] = arch


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        known = ", ".join(sorted(_ARCHITECTURES)) or "(none)"
        raise ConfigError(f"unknown architecture {name!r}; registered: {known}") from None


def registered_architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def load_model_config(folder: str) -> ModelConfig:
    raw = read_config_json(folder)
    return get_architecture(architecture_name(raw)).config_from_dict(raw)


def _ensure_builtin() -> None:
    # Imported lazily so that ``config`` does not depend on ``models`` at import time.
    from .. import models  # noqa: F401  (registers the built-in architectures)
