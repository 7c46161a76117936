"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * gain  (stratum/native/stratum_arch_llama.inc.c:45-76)."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import kernels as K
from .base import Handover, Norm
from .registry import register_part
from .spec import TensorSpec


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """params: size, eps, prefix (e.g. "input_layernorm.")."""
    replays_prompts = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.gain: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {self.prefix + "weight": TensorSpec((self.size,), role="vector", init="ones")}

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        self.gain = weights[self.prefix + "weight"]

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.numel()
        out = self.runtime.empty(n, self.size)
        K.rmsnorm(x, self.gain, self.eps, out, rows)
        return out

    def handover(self) -> Optional[Handover]:
        # the matrix products that can honour it are the bfloat16 ones; sums of squares are kept per 128 columns
        if self.runtime is None or self.runtime.dtype != torch.bfloat16 or self.size % 128 != 0:
            return None
        return Handover(self.gain, self.size, self.eps)

    def forward_heads(self, x: torch.Tensor, first_col: int, n_heads: int, head_dim: int) -> None:
        if head_dim != self.size:
            raise ValueError(f"rmsnorm of size {self.size} asked to normalise heads of {head_dim}")
        K.rmsnorm_heads(x, first_col, n_heads, head_dim, self.gain, self.eps)
