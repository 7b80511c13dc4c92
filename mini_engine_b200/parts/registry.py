"""Registries of part kinds: a plan names a part by kind and gives its parameters.

``register_mixer("my_mixer", MyMixer)`` (or the feed-forward, norm and position-encoding
twins) is all that a new part needs; a plan then says ``PartSpec("my_mixer", {...})`` for
the layers that use it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

_REGISTRIES: dict[str, dict[str, Callable[..., Any]]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position_encoding": {}, "block": {},
}


@dataclass
class PartSpec:
    kind: str
    args: dict[str, Any] = field(default_factory=dict)


def _register(family: str, kind: str, factory: Callable[..., Any], replace: bool) -> None:
    reg = _REGISTRIES[family]
    if kind in reg and not replace:
        raise ValueError(f"{family} kind {kind!r} is already registered")
    reg[kind] = factory


def register_mixer(kind, factory, *, replace=False):
    _register("mixer", kind, factory, replace)


def register_feed_forward(kind, factory, *, replace=False):
    _register("feed_forward", kind, factory, replace)


def register_norm(kind, factory, *, replace=False):
    _register("norm", kind, factory, replace)


def register_position_encoding(kind, factory, *, replace=False):
    _register("position_encoding", kind, factory, replace)


def register_block(kind, factory, *, replace=False):
    """``factory(spec: BlockSpec, shared: dict) -> Block``: how a layer's norms, mixer and feed-forward are arranged
    around the residual stream (``BlockSpec.kind`` names it)."""
    _register("block", kind, factory, replace)


def build_block(spec, shared):
    reg = _REGISTRIES["block"]
    if spec.kind not in reg:
        known = ", ".join(sorted(reg)) or "(none)"
        raise ValueError(f"unknown block kind {spec.kind!r}; registered: {known}")
    return reg[spec.kind](spec, shared)


def build_part(family: str, spec: PartSpec):
    reg = _REGISTRIES[family]
    if spec.kind not in reg:
        known = ", ".join(sorted(reg)) or "(none)"
        raise ValueError(f"unknown {family} kind {spec.kind!r}; registered: {known}")
    return reg[spec.kind](**spec.args)


def registered(family: str) -> list[str]:
    return sorted(_REGISTRIES[family])
