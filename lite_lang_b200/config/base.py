"""Typed model configurations and the registry from architecture name to model.

``config.json`` names its architecture under ``architectures``; the registry
maps that name to the typed configuration class, which in turn produces the
``ModelSpec`` that the generic model is assembled from.  Nothing else in the
package knows an architecture by name.
"""

from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, List, Mapping, Type

from .spec import ModelSpec


class ConfigError(ValueError):
    """A config.json that is incomplete, inconsistent or asks for something not built."""


class ModelConfig:
    """Base of the typed configurations.  Sub-classes are dataclasses."""

    architecture: str = ""

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:
        """The config.json keys of this configuration (round-trips through from_dict)."""
        raise NotImplementedError

    def model_spec(self) -> ModelSpec:
        raise NotImplementedError

    # the standard deviations that random weights are drawn with
    def init_scales(self) -> Dict[str, float]:
        return {"matrix": 0.02, "bias": 0.02, "norm": 0.05}


_ARCHITECTURES: Dict[str, Type[ModelConfig]] = {}


def register_architecture(name: str, config_cls: Type[ModelConfig]) -> None:
    """Make ``name`` (as in config.json's ``architectures``) known to the engine."""
    _ARCHITECTURES[name] = config_cls


def known_architectures() -> List[str]:
    return sorted(_ARCHITECTURES)


def config_from_dict(d: Mapping[str, Any]) -> ModelConfig:
    archs = d.get("architectures")
    if not archs or not isinstance(archs, (list, tuple)):
        raise ConfigError(
            "config.json has no 'architectures' list; known architectures: "
            + ", ".join(known_architectures())
        )
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(
            f"architecture {name!r} is not registered; known architectures: "
            + ", ".join(known_architectures())
        )
    return _ARCHITECTURES[name].from_dict(d)


def load_config(model_path: str) -> ModelConfig:
    """Read ``model_path/config.json`` and return the typed configuration."""
    path = os.path.join(model_path, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {model_path!r}")
    with open(path, "r", encoding="utf-8") as fh:
        return config_from_dict(json.load(fh))


def _require(d: Mapping[str, Any], key: str, typ: Callable[[Any], Any], arch: str):
    if key not in d or d[key] is None:
        raise ConfigError(f"{arch}: config.json lacks the required key {key!r}")
    try:
        return typ(d[key])
    except (TypeError, ValueError) as exc:
        raise ConfigError(f"{arch}: key {key!r} has the value {d[key]!r}: {exc}") from None
