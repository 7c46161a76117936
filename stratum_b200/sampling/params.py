"""Sampling settings, with the reference's names and meanings.

temperature <= 0 is greedy; top_k 0 is off; top_p 1.0 is off; seed picks the PCG32 streams
(environment variables STRATUM_TEMP, STRATUM_TOP_K, STRATUM_TOP_P, STRATUM_SEED in the reference,
stratum/native/stratum_arch_qwen35.inc.c:17118-17125).
"""
from __future__ import annotations

import os
from dataclasses import dataclass

from .pcg32 import DEFAULT_SEED

TOP_K_CAP = 512      # most candidates a filtered draw keeps (stratum/native/stratum_arch_qwen35.inc.c:14019)


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = DEFAULT_SEED

    def __post_init__(self):
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0 (0 = off)")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1] (1 = off)")

    @property
    def greedy(self) -> bool:
        return not (self.temperature > 0.0)

    @classmethod
    def from_env(cls, env=os.environ) -> "SamplingParams":
        return cls(temperature=float(env.get("STRATUM_TEMP", 0.0)), top_k=int(env.get("STRATUM_TOP_K", 0)),
                   top_p=float(env.get("STRATUM_TOP_P", 1.0)),
                   seed=int(env.get("STRATUM_SEED", DEFAULT_SEED)))
