from .params import TOP_K_CAP, SamplingParams
from .pcg32 import DEFAULT_SEED, Pcg32
from .sampler import Sampler

__all__ = ["TOP_K_CAP", "SamplingParams", "DEFAULT_SEED", "Pcg32", "Sampler"]
