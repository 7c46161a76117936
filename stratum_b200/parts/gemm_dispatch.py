"""Which matrix-product kernel serves a given call.

float32 always takes the CUDA-core kernel with the fixed summation order (the true 32-bit
path).  bfloat16: up to SKINNY_MAX_ROWS rows of x take the weight-streaming kernel (decode
steps of one or two sequences), more rows the tcgen05 kernels of gemm_tc.cu (stream-K for
decode steps and short prompts, tiles on pairs of CTAs or on single CTAs for prompts; the
choice among those is made there, from the shapes), and any shape either refuses (rows not
16-byte aligned) falls back to the CUDA-core kernel.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .. import kernels as K

STORE, ADD_TO_F32, STORE_F32, SWIGLU = K.EPI_STORE, K.EPI_ADD_F32, K.EPI_STORE_F32, K.EPI_SWIGLU

# rows of x up to which the weight-streaming mma.sync kernel is used.  Measured in whole decode steps on the
# Llama-8B layer shapes: one and two rows are faster with it (one kernel, no second pass), from four rows on the
# stream-K tcgen05 kernel wins (3.96 against 4.10 ms at four rows).  STRATUM_SKINNY_MAX_ROWS overrides it for
# measurements.
SKINNY_MAX_ROWS = int(os.environ.get("STRATUM_SKINNY_MAX_ROWS", 2))
# weight matrices of at least this many elements go to the stream-K kernel even for few rows of x: its TMA
# ring keeps more bytes in flight, which pays once the matrix is large enough to amortise its set-up
STREAMK_MIN_WEIGHTS = int(os.environ.get("STRATUM_STREAMK_MIN_WEIGHTS", 400_000_000))


def _aligned(x: torch.Tensor, w: torch.Tensor) -> bool:
    k = w.shape[1]
    return (k % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def run(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, mode: int) -> None:
    """out (=|+=) epilogue(x @ w.T + bias); see the EPI_* modes in kernels.py."""
    if x.dtype == torch.bfloat16 and _aligned(x, w):
        if x.shape[0] <= SKINNY_MAX_ROWS and w.numel() < STREAMK_MIN_WEIGHTS:
            K.gemm_skinny(x, w, bias, out, mode)
        else:
            K.gemm_tc(x, w, bias, out, mode)
        return
    if mode == SWIGLU:
        gu = torch.empty((x.shape[0], w.shape[0]), dtype=x.dtype, device=x.device)
        K.linear_simple(x, w, bias, gu, STORE)
        K.swiglu(gu, out)
        return
    K.linear_simple(x, w, bias, out, mode)
