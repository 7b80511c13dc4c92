"""Typed model configuration read from an architecture's own ``config.json`` keys.

The reference reads the same keys through a ``transformers`` config object that it
uses duck-typed (config.py:25, models/qwen3.py:15-17,81-84,107-108).  Here the file
is parsed directly: every size and constant of the model comes from it, none is
written in code.  A key the engine cannot honour (an activation other than SiLU,
biased projections, scaled rotary embeddings) is refused with a clear error
instead of being ignored.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, asdict
from typing import Any


class ConfigError(ValueError):
    """A config.json that is missing a key, or asks for what the engine does not do."""


def read_config_json(folder: str) -> dict[str, Any]:
    path = os.path.join(os.path.expanduser(folder), "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {folder!r}")
    with open(path) as f:
        raw = json.load(f)
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be a JSON object")
    return raw


def architecture_name(raw: dict[str, Any]) -> str:
    archs = raw.get("architectures")
    if not archs or not isinstance(archs, list) or not isinstance(archs[0], str):
        raise ConfigError("config.json has no 'architectures': [name] entry")
    return archs[0]


def _need(raw: dict, key: str, kind):
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json lacks required key {key!r}")
    v = raw[key]
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"config.json key {key!r} must be an integer, got {v!r}")
        return v
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json key {key!r} must be a number, got {v!r}")
        return float(v)
    return v


@dataclass
class ModelConfig:
    """What every architecture's configuration offers to the engine."""

    architecture: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    max_position_embeddings: int
    eos_token_id: int = -1

    def to_json_dict(self) -> dict[str, Any]:
        raise NotImplementedError


@dataclass
class Qwen3Config(ModelConfig):
    """Qwen3 dense decoder (models/qwen3.py:12-116 in the reference).

    ``head_dim`` is independent of ``hidden_size / num_attention_heads``
    (models/qwen3.py:17).  ``layer_types`` and ``sliding_window`` are config.json keys
    of this architecture that the reference never reads (all its layers attend to
    every key); here a layer whose type is ``"sliding_attention"`` attends to the last
    ``sliding_window`` keys, itself included, when ``use_sliding_window`` is true.
    """

    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0
    rms_norm_eps: float = 0.0
    rope_theta: float = 0.0
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: int | None = None
    layer_types: list[str] = field(default_factory=list)

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "Qwen3Config":
        H = _need(raw, "hidden_size", int)
        nh = _need(raw, "num_attention_heads", int)
        L = _need(raw, "num_hidden_layers", int)
        nkv = raw.get("num_key_value_heads")
        if nkv is None:
            nkv = nh
        hd = raw.get("head_dim")
        if hd is None:
            if H % nh:
                raise ConfigError(f"head_dim absent and hidden_size {H} is no multiple of {nh} heads")
            hd = H // nh
        # models/qwen3.py:81 reads rope_parameters["rope_theta"]; raw files carry it at top level.
        rope = raw.get("rope_parameters") or {}
        theta = rope.get("rope_theta", raw.get("rope_theta"))
        if theta is None:
            raise ConfigError("config.json lacks 'rope_theta' (top level or in 'rope_parameters')")
        scaling = raw.get("rope_scaling")
        rope_type = (scaling or {}).get("rope_type", (scaling or {}).get("type", rope.get("rope_type", "default")))
        if rope_type not in ("default", None):
            raise ConfigError(f"rope scaling {rope_type!r} is not supported (only plain rotary embeddings)")
        if raw.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"hidden_act {raw['hidden_act']!r} is not supported (only 'silu')")
        if raw.get("attention_bias", False):
            raise ConfigError("attention_bias=true is not supported (projections are bias-free)")
        use_win = bool(raw.get("use_sliding_window", False))
        window = raw.get("sliding_window")
        layer_types = raw.get("layer_types")
        if use_win:
            if not isinstance(window, int) or window < 1:
                raise ConfigError(f"use_sliding_window needs a positive integer 'sliding_window', got {window!r}")
            if layer_types is None:
                first = raw.get("max_window_layers", L)
                layer_types = ["sliding_attention" if i >= first else "full_attention" for i in range(L)]
        else:
            layer_types = ["full_attention"] * L
        if len(layer_types) != L or any(t not in ("full_attention", "sliding_attention") for t in layer_types):
            raise ConfigError(f"layer_types must name {L} layers as full_attention or sliding_attention")
        eos = raw.get("eos_token_id", -1)
        if isinstance(eos, list):
            eos = eos[0] if eos else -1
        cfg = cls(
            architecture=architecture_name(raw),
            vocab_size=_need(raw, "vocab_size", int),
            hidden_size=H,
            num_hidden_layers=L,
            max_position_embeddings=_need(raw, "max_position_embeddings", int),
            eos_token_id=-1 if eos is None else int(eos),
            num_attention_heads=nh,
            num_key_value_heads=int(nkv),
            head_dim=int(hd),
            intermediate_size=_need(raw, "intermediate_size", int),
            rms_norm_eps=_need(raw, "rms_norm_eps", float),
            rope_theta=float(theta),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            use_sliding_window=use_win,
            sliding_window=window if use_win else None,
            layer_types=list(layer_types),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for name in ("vocab_size", "hidden_size", "num_hidden_layers", "max_position_embeddings",
                     "num_attention_heads", "num_key_value_heads", "head_dim", "intermediate_size"):
            if getattr(self, name) < 1:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"{self.num_attention_heads} heads are no multiple of "
                              f"{self.num_key_value_heads} key/value heads")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even for rotary embeddings")
        if not self.rms_norm_eps > 0:
            raise ConfigError("rms_norm_eps must be positive")
        if not self.rope_theta > 0:
            raise ConfigError("rope_theta must be positive")

    def window_of_layer(self, i: int) -> int | None:
        return self.sliding_window if self.layer_types[i] == "sliding_attention" else None

    def to_json_dict(self) -> dict[str, Any]:
        d = asdict(self)
        arch = d.pop("architecture")
        d["architectures"] = [arch]
        d["hidden_act"] = "silu"
        d["attention_bias"] = False
        d["torch_dtype"] = "bfloat16"
        if not self.use_sliding_window:
            d.pop("layer_types")
        return d
