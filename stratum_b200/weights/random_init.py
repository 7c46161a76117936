"""Random-weights mode: write a model folder from a configuration and a seed.

The reference never ships weights; it generates a deterministic tiny model from
a fixed seed at test time (stratum/tools/make_tiny_model.py:1-9, :292-307:
matrices N(0, 1/sqrt(K)), norm gains U[0.5, 1)).  Here: matrices and biases
N(0, std), gains 1.0, each tensor from its own generator keyed by (seed,
tensor name), so the values of one tensor do not depend on which other
tensors exist or in which order they are made.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Mapping, Optional

import numpy as np
import torch

from ..config.base import ModelConfig
from ..parts.spec import TensorSpec
from .safetensors_io import write_safetensors

_TORCH_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def tensor_generator(seed: int, name: str) -> np.random.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    key = int.from_bytes(digest[:16], "little")
    return np.random.Generator(np.random.Philox(key=key))


def random_tensor(seed: int, name: str, spec: TensorSpec, std: float, dtype: torch.dtype) -> torch.Tensor:
    if spec.role == "index":
        raise ValueError(f"{name}: random mode cannot invent an integer table")
    if spec.init == "ones":
        t = torch.ones(spec.shape, dtype=torch.float32)
    elif spec.init == "zeros":
        t = torch.zeros(spec.shape, dtype=torch.float32)
    else:
        g = tensor_generator(seed, name)
        t = torch.from_numpy(g.standard_normal(spec.shape, dtype=np.float32)) * std
    return t.to(dtype)


def random_tensors(expected: Mapping[str, TensorSpec], seed: int, std: float,
                   dtype: torch.dtype, include_optional: bool = False) -> Dict[str, torch.Tensor]:
    return {n: random_tensor(seed, n, s, std, dtype) for n, s in expected.items()
            if include_optional or not s.optional}


def write_random_model(model_dir: str, config: ModelConfig, seed: int, std: float = 0.02,
                       dtype: Optional[str] = None) -> str:
    """Create `model_dir` with config.json and model.safetensors for `config`.

    dtype: "float32" | "bfloat16" | "float16"; default is the configuration's torch_dtype.
    """
    from ..engine.model import expected_tensors        # late: engine imports this package
    dtype = dtype or getattr(config, "torch_dtype", "float32")
    if dtype not in _TORCH_DTYPES:
        raise ValueError(f"dtype {dtype!r} not one of {sorted(_TORCH_DTYPES)}")
    os.makedirs(model_dir, exist_ok=True)
    raw = config.to_dict()
    raw["torch_dtype"] = dtype
    expected = expected_tensors(config)
    tensors = random_tensors(expected, seed, std, _TORCH_DTYPES[dtype])
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed), "std": repr(std)})
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(raw, f, indent=2)
    return model_dir
