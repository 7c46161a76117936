"""SwiGLU feed-forward: residual += Wd (silu(Wg xn) * (Wu xn))
(stratum/native/stratum_arch_llama.inc.c:550-555, stratum/native/stratum_engine.h:373-391).

Gate and up run as one matrix product over a weight whose rows alternate gate_j, up_j, so that
an output row holds (g_0, u_0, g_1, u_1, ...) and the activation reads neighbours.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .base import FeedForward
from .linear import ADD_TO_F32, SWIGLU, Linear
from .registry import register_part
from .spec import TensorSpec


def interleave_rows(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Rows a_0, b_0, a_1, b_1, ..."""
    return torch.stack([a, b], dim=1).reshape((a.shape[0] * 2,) + tuple(a.shape[1:])).contiguous()


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    """params: hidden, intermediate, bias, prefix."""
    replays_prompts = True
    takes_normed_rows = True
    hands_on = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec["hidden"])
        self.intermediate = int(spec["intermediate"])
        self.bias = bool(spec.get("bias", False))
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        p, H, F = self.prefix, self.hidden, self.intermediate
        t = {p + "gate_proj.weight": TensorSpec((F, H)), p + "up_proj.weight": TensorSpec((F, H)),
             p + "down_proj.weight": TensorSpec((H, F))}
        if self.bias:
            t.update({p + "gate_proj.bias": TensorSpec((F,), role="vector"),
                      p + "up_proj.bias": TensorSpec((F,), role="vector"),
                      p + "down_proj.bias": TensorSpec((H,), role="vector")})
        return t

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        p = self.prefix
        w = interleave_rows(weights[p + "gate_proj.weight"], weights[p + "up_proj.weight"])
        b = interleave_rows(weights[p + "gate_proj.bias"], weights[p + "up_proj.bias"]) if self.bias else None
        self.gate_up = Linear(self.runtime, w, b)
        self.down = Linear(self.runtime, weights[p + "down_proj.weight"], weights.get(p + "down_proj.bias"))

    def forward(self, xn, residual: torch.Tensor, step, emit=None) -> None:
        a = self.gate_up(xn, mode=SWIGLU)
        self.down(a, out=residual, mode=ADD_TO_F32, emit=emit)
