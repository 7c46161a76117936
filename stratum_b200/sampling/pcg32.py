"""PCG32 random streams, seeded and stepped as the reference does.

State update state*6364136223846793005 + inc, output xorshift-rotate; seeding sets state 0,
inc = (seed << 1) | 1, steps once, adds 0x853c49e6748fea9b, steps again; a uniform is
(u32 >> 8) * 2^-24; stream s of a batch is seeded with seed + s * 0x9E3779B97F4A7C15
(stratum/native/stratum_arch_qwen35.inc.c:13973-13992, :14010-14018).  One stream per request, so
a request's draws do not depend on which other requests share its batch.
"""
from __future__ import annotations

_MASK = (1 << 64) - 1
_MULT = 6364136223846793005
DEFAULT_SEED = 0x243F6A8885A308D3          # stratum/native/stratum_arch_qwen35.inc.c:17123
STREAM_STRIDE = 0x9E3779B97F4A7C15


class Pcg32:
    __slots__ = ("state", "inc")

    def __init__(self, seed: int = DEFAULT_SEED, stream: int = 0):
        seed = (seed + stream * STREAM_STRIDE) & _MASK
        self.state = 0
        self.inc = ((seed << 1) | 1) & _MASK
        self.next_u32()
        self.state = (self.state + 0x853C49E6748FEA9B) & _MASK
        self.next_u32()

    def next_u32(self) -> int:
        old = self.state
        self.state = (old * _MULT + self.inc) & _MASK
        xorshifted = (((old >> 18) ^ old) >> 27) & 0xFFFFFFFF
        rot = old >> 59
        return ((xorshifted >> rot) | (xorshifted << ((-rot) & 31))) & 0xFFFFFFFF

    def uniform(self) -> float:
        """A float32-exact value in [0, 1)."""
        return (self.next_u32() >> 8) / 16777216.0
