"""Typed reading of config.json keys, shared by every architecture's configuration.

The reference reads its model facts from file metadata into one typed struct,
with required and optional keys, defaults and range guards
(stratum/native/stratum_arch.h:266-460: NEED_U32 / OPT_U32 / OPT_F32).  The same
idea here over a JSON object: a `KeyReader` hands out typed values, remembers
what went wrong, and raises one error that lists every problem at once.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
    """config.json is missing a key, has a value of the wrong type, or an impossible size."""


_MISSING = object()


class KeyReader:
    """Typed access to a config.json object; collects problems instead of stopping at the first."""

    def __init__(self, raw: Dict[str, Any], where: str = "config.json"):
        if not isinstance(raw, dict):
            raise ConfigError(f"{where}: top level must be a JSON object")
        self.raw = raw
        self.where = where
        self.problems: List[str] = []

    # -- scalar readers ---------------------------------------------------
    def _get(self, key: str, default: Any) -> Any:
        v = self.raw.get(key, _MISSING)
        if v is _MISSING or v is None:
            if default is _MISSING:
                self.problems.append(f"missing required key '{key}'")
                return None
            return default
        return v

    def integer(self, key: str, default: Any = _MISSING, lo: int = 1, hi: int = 2**31 - 1) -> Optional[int]:
        v = self._get(key, default)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v == int(v):
                v = int(v)
            else:
                self.problems.append(f"'{key}' must be an integer, got {v!r}")
                return None
        if not (lo <= v <= hi):
            self.problems.append(f"'{key}'={v} outside [{lo}, {hi}]")
            return None
        return v

    def number(self, key: str, default: Any = _MISSING, lo: float = None, hi: float = None) -> Optional[float]:
        v = self._get(key, default)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            self.problems.append(f"'{key}' must be a number, got {v!r}")
            return None
        v = float(v)
        if v != v or v in (float("inf"), float("-inf")):
            self.problems.append(f"'{key}' must be finite")
            return None
        if (lo is not None and v < lo) or (hi is not None and v > hi):
            self.problems.append(f"'{key}'={v} outside [{lo}, {hi}]")
            return None
        return v

    def boolean(self, key: str, default: Any = _MISSING) -> Optional[bool]:
        v = self._get(key, default)
        if v is None:
            return None
        if not isinstance(v, bool):
            self.problems.append(f"'{key}' must be true or false, got {v!r}")
            return None
        return v

    def string(self, key: str, default: Any = _MISSING, choices=None) -> Optional[str]:
        v = self._get(key, default)
        if v is None:
            return None
        if not isinstance(v, str):
            self.problems.append(f"'{key}' must be a string, got {v!r}")
            return None
        if choices is not None and v not in choices:
            self.problems.append(f"'{key}'={v!r} not one of {sorted(choices)}")
            return None
        return v

    def id_list(self, key: str, vocab: Optional[int]) -> tuple:
        """A token id or a list of them (eos_token_id may be either); absent -> ()."""
        v = self.raw.get(key)
        if v is None:
            return ()
        ids = v if isinstance(v, list) else [v]
        out = []
        for t in ids:
            if isinstance(t, bool) or not isinstance(t, int) or t < 0 or (vocab and t >= vocab):
                self.problems.append(f"'{key}' holds {t!r}, not a token id below vocab_size")
                continue
            out.append(t)
        return tuple(out)

    def child(self, key: str) -> Optional["KeyReader"]:
        v = self.raw.get(key)
        if v is None:
            return None
        if not isinstance(v, dict):
            self.problems.append(f"'{key}' must be an object")
            return None
        return KeyReader(v, f"{self.where}:{key}")

    def adopt(self, sub: "KeyReader") -> None:
        self.problems.extend(f"{sub.where.split(':', 1)[-1]}.{p}" if ":" in sub.where else p
                             for p in sub.problems)

    def require(self, ok: bool, message: str) -> None:
        if not ok:
            self.problems.append(message)

    def finish(self) -> None:
        if self.problems:
            raise ConfigError(f"{self.where}: " + "; ".join(self.problems))


class ModelConfig:
    """Base of every architecture's typed configuration.

    Subclasses are dataclasses with `from_dict(raw)` (validating) and `to_dict()`
    (the architecture's own config.json keys, so a written folder reads back equal).
    """

    architecture: str = ""

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:
        raise NotImplementedError

    def describe(self) -> str:
        """One line per field, as the reference prints its config
        (stratum/native/stratum_arch.h:463-501)."""
        return "\n".join(f"  {k:<28} {v}" for k, v in self.to_dict().items())


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no such file (a model folder holds config.json and model.safetensors)")
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be a JSON object")
    return raw
