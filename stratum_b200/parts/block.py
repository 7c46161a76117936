"""Arrangements: how a layer's parts are wired around the residual stream."""
from __future__ import annotations

import torch

from ..cache.store import LayerCache
from .base import Arrangement
from .registry import register_part


@register_part("arrangement", "prenorm_residual")
class PreNormResidual(Arrangement):
    """x += mixer(norm_a(x)); x += feed_forward(norm_b(x)): each norm stands before its part, on the
    residual stream (stratum/native/stratum_arch_llama.inc.c:392-396, :524-532, :555)."""

    slots = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def forward(self, layer, x: torch.Tensor, step, cache: LayerCache) -> None:
        xn = layer.part("mixer_norm").forward(x)
        layer.part("mixer").forward(xn, x, step, cache)
        xn = layer.part("feed_forward_norm").forward(x)
        layer.part("feed_forward").forward(xn, x, step)
