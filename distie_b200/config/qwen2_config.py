"""Typed configuration of the Qwen2 dense decoder, read from ``config.json`` keys.

The checks are the ones the reference makes when it derives its dimensions
(worker/src/inference/qwen2/model.py:41-74) and its KV shape
(worker/src/inference/kv_cache.py:44-58): head counts, ``hidden_size ==
num_attention_heads * head_dim``, an even ``head_dim``, ``hidden_act == "silu"``,
the default RoPE type only (model.py:413-419) and no sliding-window layers
(model.py:58-60).  No size has a default here except the ones the reference
defaults itself.
"""

from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from typing import Any, Mapping


class ConfigError(ValueError):
    """A ``config.json`` the engine cannot run, with the offending key named."""


_REQUIRED = (
    "vocab_size",
    "hidden_size",
    "intermediate_size",
    "num_hidden_layers",
    "num_attention_heads",
    "rms_norm_eps",
)


@dataclass(frozen=True)
class Qwen2Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    max_position_embeddings: int | None = None
    use_sliding_window: bool = False
    sliding_window: int | None = None
    max_window_layers: int | None = None
    layer_types: tuple[str, ...] = ()
    eos_token_id: int | None = None
    bos_token_id: int | None = None
    initializer_range: float | None = None
    torch_dtype: str | None = None
    architectures: tuple[str, ...] = ("Qwen2ForCausalLM",)
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    @property
    def num_key_value_groups(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    # -- reading ----------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "Qwen2Config":
        missing = [key for key in _REQUIRED if key not in raw]
        if missing:
            raise ConfigError(f"config.json lacks required key(s): {', '.join(missing)}")
        heads = _positive_int(raw, "num_attention_heads")
        kv_heads = int(raw.get("num_key_value_heads") or heads)  # kv_cache.py:48
        hidden = _positive_int(raw, "hidden_size")
        if kv_heads < 1 or heads % kv_heads != 0:
            raise ConfigError(
                f"num_attention_heads ({heads}) must be a positive multiple of num_key_value_heads ({kv_heads})"
            )
        explicit = raw.get("head_dim")
        head_dim = int(explicit) if explicit else hidden // heads
        if head_dim < 1 or hidden != heads * head_dim:
            raise ConfigError(
                f"hidden_size ({hidden}) must equal num_attention_heads ({heads}) * head_dim ({head_dim})"
            )
        if head_dim % 2 != 0:
            raise ConfigError(f"head_dim ({head_dim}) must be even for rotate-half RoPE")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act: only 'silu' is supported, got {act!r}")
        layer_types = tuple(raw.get("layer_types") or ())
        if any(kind != "full_attention" for kind in layer_types):
            raise ConfigError("layer_types: sliding-window Qwen2 layers are not implemented")
        if raw.get("use_sliding_window", False):
            raise ConfigError("use_sliding_window: sliding-window Qwen2 layers are not implemented")
        layers = _positive_int(raw, "num_hidden_layers")
        if layer_types and len(layer_types) != layers:
            raise ConfigError(f"layer_types has {len(layer_types)} entries, num_hidden_layers is {layers}")
        max_pos = raw.get("max_position_embeddings")
        eos = raw.get("eos_token_id")
        if isinstance(eos, (list, tuple)):
            eos = eos[0] if eos else None
        known = {f for f in cls.__dataclass_fields__ if f != "extra"} | {"rope_parameters", "rope_scaling", "dtype"}
        return cls(
            vocab_size=_positive_int(raw, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=_positive_int(raw, "intermediate_size"),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=float(raw["rms_norm_eps"]),
            rope_theta=_rope_theta(raw),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            hidden_act=act,
            max_position_embeddings=int(max_pos) if max_pos else None,
            use_sliding_window=False,
            sliding_window=raw.get("sliding_window"),
            max_window_layers=raw.get("max_window_layers"),
            layer_types=layer_types,
            eos_token_id=int(eos) if eos is not None else None,
            bos_token_id=raw.get("bos_token_id"),
            initializer_range=float(raw["initializer_range"]) if "initializer_range" in raw else None,
            torch_dtype=raw.get("torch_dtype") or raw.get("dtype"),
            architectures=tuple(raw.get("architectures") or ("Qwen2ForCausalLM",)),
            extra={k: v for k, v in raw.items() if k not in known},
        )

    @classmethod
    def from_folder(cls, folder: str) -> "Qwen2Config":
        with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as handle:
            return cls.from_dict(json.load(handle))

    # -- writing ----------------------------------------------------------
    def to_dict(self) -> dict[str, Any]:
        out = {k: v for k, v in asdict(self).items() if k != "extra" and v is not None and v != ()}
        out["architectures"] = list(self.architectures)
        if self.layer_types:
            out["layer_types"] = list(self.layer_types)
        out.update(self.extra)
        return out


def _positive_int(raw: Mapping[str, Any], key: str) -> int:
    try:
        value = int(raw[key])
    except (TypeError, ValueError) as exc:
        raise ConfigError(f"{key} must be an integer, got {raw[key]!r}") from exc
    if value < 1:
        raise ConfigError(f"{key} must be >= 1, got {value}")
    return value


def _rope_theta(raw: Mapping[str, Any]) -> float:
    params = raw.get("rope_parameters") or {}
    if isinstance(params, Mapping):
        kind = params.get("rope_type", "default")
        if kind != "default":
            raise ConfigError(f"rope_parameters.rope_type: unsupported RoPE type {kind!r}")
        if "rope_theta" in params:
            return float(params["rope_theta"])
    scaling = raw.get("rope_scaling")
    if isinstance(scaling, Mapping) and scaling.get("rope_type", scaling.get("type", "default")) != "default":
        raise ConfigError(f"rope_scaling: unsupported RoPE type {scaling!r}")
    if "rope_theta" not in raw:
        raise ConfigError("config.json lacks required key(s): rope_theta")
    return float(raw["rope_theta"])
