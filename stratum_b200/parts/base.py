"""Interfaces of the parts a decoder layer is put together from.

A part is built from the sizes and constants in its `PartSpec` and from
nothing else: it does not know which model or which layer it is in.  It
declares the weight tensors it expects (`tensors()`), receives them
(`bind()`), and computes (`forward`).  Constructing a part allocates nothing
on a device, so a model's tensor list can be made on a machine without a GPU.

Data conventions during a step:
  * the residual stream `x` is float32 [tokens, hidden];
  * norms turn it into the compute dtype (`runtime.dtype`) for the matrix products;
  * a mixer or feed-forward adds its output into the residual stream in place.
"""
from __future__ import annotations

from typing import Any, Dict, Mapping, Optional

import torch

from ..cache.store import CacheSpec, LayerCache
from .spec import PartSpec, TensorSpec


class Runtime:
    """Where and in which dtype a model computes."""

    def __init__(self, dtype: torch.dtype, device):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16, not {dtype}")
        self.dtype = dtype
        self.device = torch.device(device)

        self._scratch: Dict[str, torch.Tensor] = {}

    def empty(self, *shape: int, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)

    def scratch(self, name: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """A named scratch buffer of at least `numel` elements that lives as long as the runtime
        (kernels that need global memory beyond their inputs and outputs take it from here)."""
        t = self._scratch.get(name)
        if t is None or t.numel() < numel or t.dtype != dtype:
            t = torch.empty(max(numel, 1), dtype=dtype, device=self.device)
            self._scratch[name] = t
            from .. import kernels
            kernels.scratch_regrown()
        return t


class NormedRows:
    """Rows that a norm hands to a matrix product without writing them out in full.

    `x` [rows, size] holds r * gain in the compute dtype (r: the residual rows); `ss` float32 [parts or more, rows]
    holds partial sums of r^2, to be added in the order of the parts.  The product multiplies its result rows by
    1 / sqrt(sum / size + eps), which is what the norm would have multiplied the operand rows by.  They are made
    by the matrix product that wrote the residual rows (see Handover), so the norm costs no pass over memory."""

    def __init__(self, x: torch.Tensor, ss: torch.Tensor, parts: int, size: int, eps: float):
        self.x, self.ss, self.parts, self.size, self.eps = x, ss, parts, size, eps

    @property
    def shape(self):
        return self.x.shape


class Handover:
    """A norm's request to the part in front of it: "with the matrix product that adds your result into the
    residual stream, also leave what I need" (gain, size, eps).  A part that honours it sets `result` to the
    NormedRows; one that does not leaves it None, and the norm runs as a kernel of its own."""

    def __init__(self, gain: torch.Tensor, size: int, eps: float):
        self.gain, self.size, self.eps = gain, size, eps
        self.result: Optional[NormedRows] = None


class Part:
    kind = ""
    takes_normed_rows = False    # forward accepts NormedRows in place of the normed tensor
    hands_on = False             # forward takes `emit=Handover` and may honour it
    # forward also serves a captured prompt step (engine/graphs.py, PromptGraphs): beside the rules for captured
    # decode steps, tokens with sequence index -1 belong to no sequence (nothing of theirs reaches a cache or a
    # state row), sequences may bring no token, and query blocks come from step.query_blocks only.  A model whose
    # parts and arrangements all say so has its short prompt steps replayed; others run them launch by launch.
    replays_prompts = False

    def __init__(self, spec: PartSpec, runtime: Optional[Runtime]):
        self.spec = spec
        self.runtime = runtime
        self.prefix: str = spec.get("prefix", "")

    def tensors(self) -> Dict[str, TensorSpec]:
        """Expected weights, by name relative to the layer (the part's own prefix included)."""
        return {}

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        """Receive the tensors named by `tensors()` (optional ones may be absent)."""


class Norm(Part):
    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """float32 [T, hidden] -> compute dtype [T or len(rows), hidden]."""
        raise NotImplementedError

    def handover(self) -> Optional[Handover]:
        """A request for the part in front of this norm (see Handover), or None if this norm cannot be handed over."""
        return None

    def forward_heads(self, x: torch.Tensor, first_col: int, n_heads: int, head_dim: int) -> None:
        """Normalise in place, in every row of x (compute dtype), each of the n_heads stretches of head_dim
        values that start at column first_col: the form a mixer uses on its queries and keys.  Optional."""
        raise NotImplementedError(f"norm {self.kind!r} has no per-head form")


class PositionEncoding(Part):
    def rotary(self) -> Optional["RotaryTable"]:
        """Frequencies for a mixer that rotates queries and keys, or None if this encoding does not rotate."""
        return None

    def pair_layout(self):
        """(number of rotated pairs, interleaved) of a rotating encoding, or None; asked for when weights are
        bound and when a model is only described, so it must not need a device."""
        rot = self.rotary()
        return None if rot is None else (int(rot.inv_freq.numel()), bool(rot.interleaved))

    def add_to_embedding(self, x: torch.Tensor, step) -> None:
        """Hook for encodings that act on the embedded tokens; the default does nothing."""


class RotaryTable:
    """inv_freq: float32 [n_pairs] on the device; pairs (2k,2k+1) if interleaved else (k, k+n_pairs)."""

    def __init__(self, inv_freq: torch.Tensor, interleaved: bool, magnitude: float = 1.0, key=None):
        self.inv_freq = inv_freq
        self.interleaved = interleaved
        self.magnitude = magnitude
        # tables with equal keys rotate alike: a step evaluates the angles of its tokens once per key, not once
        # per layer (default: a key of this table's own)
        self.key = key if key is not None else ("table", id(self))


class Mixer(Part):
    def cache_spec(self) -> Optional[CacheSpec]:
        """What this mixer keeps per sequence between steps (keys and values, fixed-size state, nothing)."""
        return None

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, step, cache: LayerCache) -> None:
        """residual += mix(xn).  xn: compute dtype [T, hidden]; residual: float32 [T, hidden]."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, xn: torch.Tensor, residual: torch.Tensor, step) -> None:
        """residual += ffn(xn)."""
        raise NotImplementedError


class Embedding(Part):
    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        """int32 [T] -> float32 [T, hidden]."""
        raise NotImplementedError

    def table(self) -> torch.Tensor:
        raise NotImplementedError


class Head(Part):
    def bind_with_embedding(self, weights: Mapping[str, torch.Tensor], table: torch.Tensor) -> None:
        self.bind(weights)

    def forward(self, xn: torch.Tensor) -> torch.Tensor:
        """compute dtype [n, hidden] -> float32 logits [n, vocab]."""
        raise NotImplementedError


class Arrangement:
    """How a layer's parts are wired around the residual stream.

    `slots` names the parts this arrangement uses and the category each is looked up in; a layer's spec must
    give exactly those (names in `optional` may be left out).  `cache_owner` names the part whose
    `cache_spec()` says what the layer keeps per sequence (None: nothing).  `forward` reads the built parts
    as `layer.part(name)`."""
    kind = ""
    slots: Mapping[str, str] = {}
    optional: tuple = ()
    cache_owner: Optional[str] = "mixer"
    carries = False     # forward takes carry= / hand_to= and returns a carry (see accepts_carry)
    replays_prompts = False    # as Part.replays_prompts

    def forward(self, layer, x: torch.Tensor, step, cache: LayerCache) -> None:
        raise NotImplementedError

    def accepts_carry(self, layer) -> Optional["Norm"]:
        """The norm this layer begins with, if the layer can begin from NormedRows made for that norm by the
        layer in front of it (then the model passes them as `carry=` and asks the layer in front with
        `hand_to=` that norm); None otherwise."""
        return None
