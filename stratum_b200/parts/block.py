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
    replays_prompts = True

    slots = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}
    carries = True

    def accepts_carry(self, layer):
        return layer.part("mixer_norm") if layer.part("mixer").takes_normed_rows else None

    def forward(self, layer, x: torch.Tensor, step, cache: LayerCache, carry=None, hand_to=None):
        """carry: NormedRows of x made for this layer's first norm by the layer before (or None).  hand_to: the
        norm the next layer begins with, if it can begin from NormedRows; they are returned (or None).
        A norm whose rows were handed over runs no kernel: the product in front of it left what it needs."""
        norm_a, mixer = layer.part("mixer_norm"), layer.part("mixer")
        norm_b, ff = layer.part("feed_forward_norm"), layer.part("feed_forward")
        xn = carry if carry is not None else norm_a.forward(x)
        ask = norm_b.handover() if mixer.hands_on and ff.takes_normed_rows else None
        if ask is not None:
            mixer.forward(xn, x, step, cache, emit=ask)
        else:
            mixer.forward(xn, x, step, cache)
        xn = ask.result if ask is not None and ask.result is not None else norm_b.forward(x)
        ask = hand_to.handover() if hand_to is not None and ff.hands_on else None
        if ask is not None:
            ff.forward(xn, x, step, emit=ask)
            return ask.result
        ff.forward(xn, x, step)
        return None
