"""Data that describes a model: which parts, with which sizes, in which order.

An architecture turns its typed configuration into a `ModelSpec`; the engine
builds the parts named there from the part registry.  Nothing in a spec is
code: a layer names its mixer, feed-forward, norms and arrangement by kind,
with their sizes and constants as parameters, so two layers of one model may
use different kinds; and the order in which layers run is a list of its own.

The reference classifies layers per index from its configuration
(stratum/native/stratum_arch.h:82-105: full attention / SSM / next-token
layers); this is the same idea with open-ended kinds.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: its registered kind and its sizes and constants."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: an arrangement and the parts it wires, by the names the arrangement gives them.

    `parts` maps a name to a PartSpec.  Which names exist, and of which category each is (mixer, norm,
    feed_forward, ...), is the arrangement's business: "prenorm_residual" asks for `mixer_norm`, `mixer`,
    `feed_forward_norm` and `feed_forward`; another arrangement may ask for one shared norm, for four, or
    for no feed-forward at all.  Tensor names are the layer's prefix, then the part's own prefix.
    """
    arrangement: str                 # registered arrangement kind, e.g. "prenorm_residual"
    parts: Mapping[str, PartSpec]
    prefix: str                      # tensor-name prefix of this layer's weights


@dataclass(frozen=True)
class ScheduleEntry:
    """One stop of the forward pass.

    `layer` indexes ModelSpec.layers; a layer may appear at more than one stop (its weights are
    shared, each stop keeps a cache of its own).
    `cache_of`: the earlier stop (its position in the schedule) whose cache this stop reads; None
    means its own.  A stop that reads another stop's cache writes no keys or state of its own.
    """
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    hidden: int
    vocab: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    position: Optional[PartSpec] = None     # an encoding that acts on the embedded tokens (absolute positions)

    def check(self) -> None:
        n = len(self.layers)
        if not self.schedule:
            raise ValueError("model spec: empty schedule")
        for i, e in enumerate(self.schedule):
            if not (0 <= e.layer < n):
                raise ValueError(f"model spec: schedule names layer {e.layer}, model has {n}")
            if e.cache_of is not None:
                if not (0 <= e.cache_of < i):
                    raise ValueError(f"model spec: stop {i} reads the cache of stop {e.cache_of}, which is not earlier")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(f"model spec: stop {i} reads the cache of stop {e.cache_of}, which has none of its own")


@dataclass(frozen=True)
class TensorSpec:
    """A weight tensor a part expects: its shape and what it is used as.

    role: "matrix"  - an operand of a matrix product or an embedding table; kept in the
                      compute dtype (bfloat16 on the bfloat16 path);
          "vector"  - gains and biases; always held in float32 (exact from bfloat16);
          "keep"    - held in the dtype the file stores (float32 stays float32);
          "index"   - integer table, held as int32.
    init: how random-weights mode fills it: "normal" (std from the caller), "ones", "zeros".
    optional: absence is not an error (the part then does without it).
    """
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    optional: bool = False
