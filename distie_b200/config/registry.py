"""One registry from an architecture's name to its configuration class and recipe.

The reference hard-codes its one model (worker/src/inference/torch_engine.py:142);
here the name in ``config.json["architectures"][0]`` selects an entry, everywhere:
the loader, the random-weights writer, generation and trace replay.

An entry is ``(config_cls, recipe)``: ``config_cls.from_dict(raw_json)`` gives the
typed configuration and ``recipe(config)`` gives the
:class:`~distie_b200.config.model_spec.ModelSpec` the rest of the engine builds from.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Mapping

from .model_spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: Any
    recipe: Callable[[Any], ModelSpec]


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: Any, recipe: Callable[[Any], ModelSpec]) -> Architecture:
    entry = Architecture(name, config_cls, recipe)
    _ARCHITECTURES[name] = entry
    return entry


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures() -> tuple[str, ...]:
    _load_builtin()
    return tuple(sorted(_ARCHITECTURES))


def get_architecture(name: str) -> Architecture:
    _load_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise KeyError(
            f"unknown architecture {name!r}; registered: {', '.join(sorted(_ARCHITECTURES)) or '(none)'}"
        ) from None


def architecture_of(raw: Mapping[str, Any]) -> Architecture:
    names = raw.get("architectures") or ()
    if not names:
        raise KeyError("config.json has no 'architectures' entry to choose a model by")
    return get_architecture(names[0])


def read_config(folder: str):
    """``(architecture, typed config)`` of the model folder."""
    path = os.path.join(folder, "config.json")
    with open(path, "r", encoding="utf-8") as handle:
        raw = json.load(handle)
    arch = architecture_of(raw)
    return arch, arch.config_cls.from_dict(raw)


def _load_builtin() -> None:
    # The built-in recipes register themselves on import.
    from .. import models  # noqa: F401
