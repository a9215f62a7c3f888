"""One registry from an architecture's name (config.json ``architectures[0]``) to its model.

An entry holds the typed configuration class that parses the architecture's config.json keys
and the function that turns that configuration into a ``ModelSpec``.  The reference has no
registry: ``Engine.from_pretrained`` hard-codes its one model class (engine/engine.py:130).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping

from .model_config import ConfigError, ModelConfig, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Mapping[str, Any]], ModelConfig]
    build_spec: Callable[[ModelConfig], Any]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(
    name: str,
    parse_config: Callable[[Mapping[str, Any]], ModelConfig],
    build_spec: Callable[[ModelConfig], Any],
) -> None:
    _ARCHITECTURES[name] = Architecture(name, parse_config, build_spec)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def supported_architectures():
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    _load_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"architecture {name!r} is not supported; supported: {supported_architectures()}"
        ) from None


def architecture_of(config_json: Mapping[str, Any]) -> Architecture:
    names = config_json.get("architectures")
    if not names or not isinstance(names, (list, tuple)):
        raise ConfigError("config.json has no 'architectures' list to choose the model by")
    return get_architecture(str(names[0]))


def load_model_config(model_dir: str) -> ModelConfig:
    """Read ``model_dir/config.json`` into the typed configuration of its architecture."""
    raw = read_config_json(model_dir)
    return architecture_of(raw).parse_config(raw)


def _load_builtin() -> None:
    # Importing the models package registers the built-in architectures.
    from .. import models  # noqa: F401
