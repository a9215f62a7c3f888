"""Registries of part classes, by kind and name.

A part class is registered under a kind ("mixer", "feed_forward", "norm", "position", "block",
"embedding", "lm_head") and a name; a ``PartSpec`` names it by that name.  Registering a class
is all it takes to make it usable from a model spec: code outside this package (a test, an
extension) can add a mixer without touching any file here.
"""
from __future__ import annotations

from typing import Callable, Dict, Type

KINDS = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "lm_head")

_REGISTRY: Dict[str, Dict[str, type]] = {kind: {} for kind in KINDS}


def register_part(kind: str, name: str) -> Callable[[type], type]:
    if kind not in _REGISTRY:
        raise ValueError(f"unknown part kind {kind!r}; expected one of {KINDS}")

    def decorator(cls: type) -> type:
        known = _REGISTRY[kind].get(name)
        if known is not None and known is not cls:
            raise ValueError(f"{kind} {name!r} is already registered as {known.__name__}")
        _REGISTRY[kind][name] = cls
        return cls

    return decorator


def unregister_part(kind: str, name: str) -> None:
    _REGISTRY[kind].pop(name, None)


def part_class(kind: str, name: str) -> Type:
    try:
        return _REGISTRY[kind][name]
    except KeyError:
        raise KeyError(
            f"no {kind} named {name!r} is registered; known: {sorted(_REGISTRY.get(kind, {}))}"
        ) from None
