"""One registry per category of part: name -> class.

A part registers itself under a category ("mixer", "feed_forward", "norm",
"position", "arrangement", "embedding", "head").  A model spec refers to
parts only by these names, so a new part needs no change to the engine: define
the class, register it, name it in a spec.  The reference registers whole
architectures the same way, by name in a table
(stratum/native/stratum_arch.h:120-187).
"""
from __future__ import annotations

from typing import Callable, Dict, Type

CATEGORIES = ("mixer", "feed_forward", "norm", "position", "arrangement", "embedding", "head")

_REGISTRY: Dict[str, Dict[str, type]] = {c: {} for c in CATEGORIES}


def register_part(category: str, name: str, *, replace: bool = False) -> Callable[[type], type]:
    if category not in _REGISTRY:
        raise KeyError(f"unknown part category {category!r}; categories: {list(CATEGORIES)}")

    def deco(cls: type) -> type:
        if name in _REGISTRY[category] and not replace and _REGISTRY[category][name] is not cls:
            raise KeyError(f"{category} {name!r} is already registered")
        _REGISTRY[category][name] = cls
        cls.kind = name
        return cls

    return deco


def find_part(category: str, name: str) -> type:
    try:
        return _REGISTRY[category][name]
    except KeyError:
        known = ", ".join(sorted(_REGISTRY.get(category, {}))) or "(none)"
        raise KeyError(f"no {category} named {name!r}; registered: {known}") from None


def registered(category: str):
    return sorted(_REGISTRY[category])
