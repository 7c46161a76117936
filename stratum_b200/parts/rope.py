"""Rotary position encoding: the frequency table and its long-context rescalings.

inv_k = 1 / theta^(2k / rope_dim), k < rope_dim/2, computed in float32 as the reference does
(stratum/native/stratum_arch_llama.inc.c:114-129); the angle of position p is (float)p * inv_k,
evaluated inside the kernel that rotates.  Rescalings, applied once when the table is built
(as the reference does for its own types, stratum/native/stratum_rope.h:82-112):
  linear: inv_k / factor
  yarn:   ramp between inv_k and inv_k / factor over the corrected dimension range, and a
          magnitude factor 0.1 ln(factor) + 1 on cos and sin
  llama3: by wavelength L = 2 pi / inv_k:  L < orig/high -> inv_k;  L > orig/low -> inv_k/factor;
          between: s = (orig/L - low)/(high - low), (1-s) inv_k/factor + s inv_k   (not in the
          reference; the published Llama-3.1 rule)
Pair layout is a parameter: (k, k + n_pairs) for weights in the safetensors convention,
(2k, 2k+1) for the reference's GGUF "llama" convention (stratum/native/stratum_arch_llama.inc.c:82-87).
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch

from .base import PositionEncoding, RotaryTable
from .registry import register_part


def inverse_frequencies(rope_dim: int, theta: float, scaling: Optional[dict]) -> (np.ndarray, float):
    """float32 inv_freq [rope_dim/2] and the magnitude factor for cos/sin."""
    n_pairs = rope_dim // 2
    k = np.arange(n_pairs, dtype=np.float32)
    base = (np.float32(1.0) / np.power(np.float32(theta), (2.0 * k / np.float32(rope_dim)).astype(np.float32))
            ).astype(np.float32)
    kind = (scaling or {}).get("kind", "none")
    if kind in ("none", "default"):
        return base, 1.0
    factor = float(scaling["factor"])
    if not factor > 1.0:
        return base, 1.0
    if kind == "linear":
        return (base / np.float32(factor)).astype(np.float32), 1.0
    if kind == "llama3":
        low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
        orig = float(scaling["original_max_position"])
        out = base.astype(np.float64)
        for i, f in enumerate(base.astype(np.float64)):
            lam = 2.0 * math.pi / f
            if lam < orig / high:
                out[i] = f
            elif lam > orig / low:
                out[i] = f / factor
            else:
                s = (orig / lam - low) / (high - low)
                out[i] = (1.0 - s) * f / factor + s * f
        return out.astype(np.float32), 1.0
    if kind == "yarn":
        orig = float(scaling["original_max_position"])
        beta_fast, beta_slow = float(scaling.get("beta_fast", 32.0)), float(scaling.get("beta_slow", 1.0))
        dim = float(rope_dim)

        def corr(n_rot: float) -> float:
            return dim * math.log(orig / (n_rot * 2.0 * math.pi)) / (2.0 * math.log(theta))

        lo = max(0.0, math.floor(corr(beta_fast)))
        hi = min(dim - 1.0, math.ceil(corr(beta_slow)))
        denom = max(hi - lo, 0.001)
        out = np.empty_like(base)
        for i in range(n_pairs):
            y = min(1.0, max(0.0, (i - lo) / denom))
            ramp = 1.0 - y
            out[i] = np.float32(base[i] / factor * (1.0 - ramp) + base[i] * ramp)
        att = float(scaling.get("attention_factor", -1.0))
        return out, (att if att > 0 else 0.1 * math.log(factor) + 1.0)
    raise ValueError(f"unknown rope scaling kind {kind!r}")


@register_part("position", "rope")
class RotaryEmbedding(PositionEncoding):
    """params: rope_dim, theta, interleaved, scaling (dict with 'kind' and its numbers, or None)."""
    replays_prompts = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.rope_dim = int(spec["rope_dim"])
        self.theta = float(spec["theta"])
        self.interleaved = bool(spec.get("interleaved", False))
        self.scaling = spec.get("scaling")
        self._table: Optional[RotaryTable] = None

    def pair_layout(self):
        return self.rope_dim // 2, self.interleaved

    def rotary(self) -> RotaryTable:
        if self._table is None:
            inv, mag = inverse_frequencies(self.rope_dim, self.theta, self.scaling)
            key = ("rope", self.rope_dim, self.theta, self.interleaved,
                   tuple(sorted((self.scaling or {}).items())), str(self.runtime.device))
            self._table = RotaryTable(torch.from_numpy(inv).to(self.runtime.device), self.interleaved, mag, key)
        return self._table


@register_part("position", "none")
class NoPositionEncoding(PositionEncoding):
    """Queries and keys are used as projected."""
    replays_prompts = True
