"""Token embedding (a row gather, stratum/native/stratum_arch_llama.inc.c:564-593) and the output
head (logits = W xn with W the head's own matrix if the file has one, else the embedding table,
stratum/native/stratum_arch_llama.inc.c:722-723)."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import kernels as K
from .base import Embedding, Head
from .linear import STORE_F32, Linear
from .registry import register_part
from .spec import TensorSpec


@register_part("embedding", "token_embedding")
class TokenEmbedding(Embedding):
    """params: vocab, hidden, prefix (e.g. "model.embed_tokens.")."""
    replays_prompts = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab, self.hidden = int(spec["vocab"]), int(spec["hidden"])
        self._table: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {self.prefix + "weight": TensorSpec((self.vocab, self.hidden))}

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        self._table = weights[self.prefix + "weight"]

    def table(self) -> torch.Tensor:
        return self._table

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        out = self.runtime.empty(token_ids.numel(), self.hidden, dtype=torch.float32)
        K.embed_gather(self._table, token_ids, out)
        return out


@register_part("head", "linear_head")
class LinearHead(Head):
    """params: vocab, hidden, tied (the file may leave the matrix out), prefix (e.g. "lm_head.")."""
    replays_prompts = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab, self.hidden = int(spec["vocab"]), int(spec["hidden"])
        self.tied = bool(spec.get("tied", False))
        self.proj: Optional[Linear] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {self.prefix + "weight": TensorSpec((self.vocab, self.hidden), optional=self.tied)}

    def bind_with_embedding(self, weights: Mapping[str, torch.Tensor], table: torch.Tensor) -> None:
        w = weights.get(self.prefix + "weight")
        self.proj = Linear(self.runtime, w if w is not None else table)

    def forward(self, xn: torch.Tensor) -> torch.Tensor:
        return self.proj(xn, mode=STORE_F32)
