"""A model built from a ModelSpec: parts, their weights, and the forward pass over one step.

The model class is chosen by config.json through the architecture registry; from there on
everything is generic: the spec names parts, the part registry builds them, the schedule says
in which order layers run and whose cache each stop uses.
"""
from __future__ import annotations

import hashlib
import os
from typing import Dict, List, Mapping, Optional, Tuple

import torch

from .. import architectures  # noqa: F401  (registers the built-in architectures)
from ..cache.store import CacheSpec
from ..config.base import ModelConfig, read_config_json
from ..config.registry import find_architecture
from ..parts import find_part
from ..parts.base import Runtime
from ..parts.spec import LayerSpec, ModelSpec, TensorSpec
from ..weights.loader import check_tensors, load_weights, place


class Layer:
    """The parts of one decoder layer, built from its LayerSpec: whichever the arrangement asks for."""

    def __init__(self, spec: LayerSpec, runtime: Optional[Runtime]):
        self.spec = spec
        self.prefix = spec.prefix
        self.arrangement = find_part("arrangement", spec.arrangement)()
        slots, optional = self.arrangement.slots, set(self.arrangement.optional)
        missing = [n for n in slots if n not in spec.parts and n not in optional]
        unknown = [n for n in spec.parts if n not in slots]
        if missing or unknown:
            raise ValueError(f"layer {spec.prefix!r}: arrangement {spec.arrangement!r} wires the parts "
                             f"{sorted(slots)}; missing {missing}, not known to it {unknown}")
        self._parts: Dict[str, object] = {name: find_part(slots[name], ps.kind)(ps, runtime)
                                          for name, ps in spec.parts.items()}

    def part(self, name: str):
        """The built part of that name, or None when the spec left an optional one out."""
        return self._parts.get(name)

    def parts(self):
        return tuple(self._parts.values())

    def cache_spec(self) -> Optional[CacheSpec]:
        owner = self.arrangement.cache_owner
        part = self._parts.get(owner) if owner else None
        return part.cache_spec() if part is not None else None

    def tensors(self) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for p in self.parts():
            for name, ts in p.tensors().items():
                out[self.prefix + name] = ts
        return out

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        n = len(self.prefix)
        local = {k[n:]: v for k, v in weights.items() if k.startswith(self.prefix)}
        for p in self.parts():
            p.bind(local)


class Model:
    """Parts of a whole model.  Without a runtime it only describes (tensor list, cache needs)."""

    def __init__(self, spec: ModelSpec, runtime: Optional[Runtime]):
        spec.check()
        self.spec = spec
        self.runtime = runtime
        self.embedding = find_part("embedding", spec.embedding.kind)(spec.embedding, runtime)
        self.layers: List[Layer] = [Layer(ls, runtime) for ls in spec.layers]
        self.final_norm = find_part("norm", spec.final_norm.kind)(spec.final_norm, runtime)
        self.head = find_part("head", spec.head.kind)(spec.head, runtime)
        self.position = (find_part("position", spec.position.kind)(spec.position, runtime)
                         if spec.position is not None else None)
        self.schedule = spec.schedule
        self.hidden, self.vocab = spec.hidden, spec.vocab

    # ------------------------------------------------------------------ description
    def tensors(self) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        out.update(self.embedding.tensors())
        if self.position is not None:
            out.update(self.position.tensors())
        for layer in self.layers:
            out.update(layer.tensors())
        out.update(self.final_norm.tensors())
        out.update(self.head.tensors())
        return out

    def cache_specs(self) -> List[Optional[CacheSpec]]:
        """Per stop of the schedule: what its mixer keeps per sequence (None if nothing, or if the stop
        reads another stop's cache)."""
        specs: List[Optional[CacheSpec]] = []
        for i, e in enumerate(self.schedule):
            own = self.layers[e.layer].cache_spec()
            if e.cache_of is not None:
                theirs = self.layers[self.schedule[e.cache_of].layer].cache_spec()
                if theirs != own:
                    raise ValueError(f"model spec: stop {i} needs {own} but reads the cache of stop {e.cache_of}, "
                                     f"which holds {theirs}")
                own = None
            specs.append(own)
        return specs

    # ------------------------------------------------------------------ weights
    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        self.embedding.bind(weights)
        if self.position is not None:
            self.position.bind(weights)
        for layer in self.layers:
            layer.bind(weights)
        self.final_norm.bind(weights)
        self.head.bind_with_embedding(weights, self.embedding.table())

    def replays_prompts(self) -> bool:
        """Whether every part and arrangement serves captured prompt steps (Part.replays_prompts)."""
        parts = [self.embedding, self.final_norm, self.head] + ([self.position] if self.position is not None else [])
        for layer in self.layers:
            parts += list(layer.parts()) + [layer.arrangement]
        return all(getattr(p, "replays_prompts", False) for p in parts)

    # ------------------------------------------------------------------ forward
    def forward(self, step, cache) -> torch.Tensor:
        """Run the tokens of one step through every stop of the schedule; float32 logits at the wanted rows."""
        x = self.embedding.forward(step.token_ids)
        if self.position is not None:
            self.position.add_to_embedding(x, step)
        carry = None                  # rows a layer's last product prepared for the next layer's first norm
        for stop, entry in enumerate(self.schedule):
            layer = self.layers[entry.layer]
            owner = stop if entry.cache_of is None else entry.cache_of
            view = cache.layer_view(owner, entry.cache_of is None, step.block_tables)
            if layer.arrangement.carries:
                hand_to = None
                if stop + 1 < len(self.schedule):
                    nxt = self.layers[self.schedule[stop + 1].layer]
                    hand_to = nxt.arrangement.accepts_carry(nxt) if nxt.arrangement.carries else None
                carry = layer.arrangement.forward(layer, x, step, view, carry=carry, hand_to=hand_to)
            else:
                layer.arrangement.forward(layer, x, step, view)
                carry = None
        if step.want_rows.numel() == 0:
            return torch.empty((0, self.vocab), dtype=torch.float32, device=x.device)
        xn = self.final_norm.forward(x, rows=step.want_rows)
        return self.head.forward(xn)


def config_from_dir(model_dir: str) -> Tuple[ModelConfig, object]:
    raw = read_config_json(model_dir)
    arch = find_architecture(raw)
    return arch.config_class.from_dict(raw), arch


def expected_tensors(config: ModelConfig) -> Dict[str, TensorSpec]:
    """Every tensor a model of this configuration expects; needs no GPU."""
    arch = find_architecture(config.architecture)
    return Model(arch.describe_model(config), None).tensors()


def load_model(model_dir: str, dtype: torch.dtype, device="cuda") -> Tuple[Model, ModelConfig]:
    """config.json picks the architecture; weights are bound by name."""
    config, arch = config_from_dir(model_dir)
    runtime = Runtime(dtype, device)
    model = Model(arch.describe_model(config), runtime)
    weights = load_weights(model_dir, model.tensors(), dtype, runtime.device, arch.ignored_tensor_suffixes)
    model.bind(weights)
    return model, config


def model_from_tensors(config: ModelConfig, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype,
                       device="cuda") -> Model:
    """Build from tensors already in memory (checked like a file's)."""
    arch = find_architecture(config.architecture)
    runtime = Runtime(dtype, device)
    model = Model(arch.describe_model(config), runtime)
    expected = model.tensors()
    check_tensors("tensors in memory", expected, tensors, arch.ignored_tensor_suffixes)
    placed = {n: place(tensors[n], s, dtype, runtime.device) for n, s in expected.items() if n in tensors}
    model.bind(placed)
    return model


def random_model_on_device(config: ModelConfig, seed: int, dtype: torch.dtype, device="cuda",
                           std: float = 0.02) -> Model:
    """Random weights made on the device by the seeded fill kernel (no files): for measurements."""
    from .. import kernels as K
    arch = find_architecture(config.architecture)
    runtime = Runtime(dtype, device)
    model = Model(arch.describe_model(config), runtime)
    weights: Dict[str, torch.Tensor] = {}
    for name, ts in model.tensors().items():
        if ts.optional:
            continue
        dt = torch.float32 if ts.role in ("vector", "keep") else dtype
        t = torch.empty(ts.shape, dtype=dt, device=runtime.device)
        if ts.init == "ones":
            t.fill_(1.0)
        elif ts.init == "zeros":
            t.zero_()
        else:
            # keyed by (seed, tensor name, element index): a tensor's values do not depend on which other
            # tensors the model has or in which order they are made
            key = int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little")
            K.fill_normal(t, key, std)
        weights[name] = t
    model.bind(weights)
    return model
