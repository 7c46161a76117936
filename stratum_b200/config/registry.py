"""Architecture registry: the name in config.json -> typed configuration and model description.

The reference keeps a table of handlers keyed by a comma-separated list of
architecture names and lists the known ones when a name is not found
(stratum/native/stratum_arch.h:120-187, stratum/native/stratum.c:81-91).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Tuple, Type

from .base import ConfigError, ModelConfig


@dataclass(frozen=True)
class Architecture:
    names: Tuple[str, ...]                       # values of `architectures[0]` / `model_type` it answers to
    description: str
    config_class: Type[ModelConfig]
    describe_model: Callable[[ModelConfig], Any]  # typed config -> parts.spec.ModelSpec
    # tensors a published file may carry that the model does not use (buffers, not weights): names ending in one
    # of these are left alone by the loader instead of being reported as unexpected
    ignored_tensor_suffixes: Tuple[str, ...] = ()


_ARCHITECTURES: List[Architecture] = []


def register_architecture(arch: Architecture, *, replace: bool = False) -> Architecture:
    for name in arch.names:
        for i, other in enumerate(_ARCHITECTURES):
            if name in other.names:
                if not replace:
                    raise KeyError(f"architecture name {name!r} is already registered")
                _ARCHITECTURES.pop(i)
                break
    _ARCHITECTURES.append(arch)
    return arch


def registered_architectures() -> List[Architecture]:
    from .. import architectures  # noqa: F401
    return list(_ARCHITECTURES)


def architecture_name(raw: Dict[str, Any]) -> str:
    archs = raw.get("architectures")
    if isinstance(archs, list) and archs and isinstance(archs[0], str):
        return archs[0]
    mt = raw.get("model_type")
    if isinstance(mt, str):
        return mt
    raise ConfigError("config.json: neither 'architectures' nor 'model_type' names the model")


def find_architecture(raw_or_name) -> Architecture:
    from .. import architectures  # noqa: F401  (the built-in architectures register themselves on import)
    name = raw_or_name if isinstance(raw_or_name, str) else architecture_name(raw_or_name)
    for arch in _ARCHITECTURES:
        if name in arch.names:
            return arch
    known = "; ".join(f"{'/'.join(a.names)} ({a.description})" for a in _ARCHITECTURES) or "(none)"
    raise ConfigError(f"no handler for architecture {name!r}; registered: {known}")
