"""Which matrix-product kernel serves a given call.

float32 always takes the CUDA-core kernel with the fixed summation order (the true 32-bit
path).  bfloat16: up to SKINNY_MAX_ROWS rows of x and a small weight matrix take the weight-streaming kernel
(decode steps of a few sequences), more rows the tcgen05 kernels of gemm_tc.cu (stream-K for
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

# rows of x up to which the weight-streaming mma.sync kernel is used, for weight matrices of fewer than
# STREAMK_MIN_WEIGHTS elements: larger ones go to the tcgen05 kernels whatever the rows, whose TMA ring keeps more
# bytes in flight.  Measured in whole decode steps of one sequence: on the Llama-8B shapes 3.36 ms with the
# threshold at 20 M elements (the output projection alone on the mma.sync kernel), 3.43 ms with every product on
# tcgen05, 3.61 ms with every product on mma.sync; on the Llama-3.2-1B shapes 0.93, 1.07 and 0.92 ms.  With four
# rows the output projection is still ahead on mma.sync (3.64 against 3.69 ms a step), with eight it makes no
# difference (4.00 against 3.99); on the Llama-3.2-1B shapes, where all but gate|up are that small, the step is
# 8 to 11 % shorter with three to eight rows (1.20 against 1.29 ms at eight) and the same with sixteen.  Both can
# be set in the environment for measurements.
# Where a product that adds into the residual stream honours the next norm's Handover (writes the bfloat16 rows
# and the sums of squares the norm needs, so that the norm runs no kernel): where its tiles of 256 x 256 fill most
# pairs of SMs, HANDOVER_MIN_TILES of them, and from HANDOVER_MIN_ROWS rows on.  Measured on the Llama-8B layer
# sizes: at 2,048 rows the two norm kernels of a layer (14 us each) go and the products' epilogues grow by
# 12 + 5 + 5 us; in decode steps the norm kernels cost nothing to begin with (they run while the next product's
# weights stream in) and the longer epilogues make a step 4 % slower.  Between: a product that hands over cannot
# share its left-over tiles along k (the second kernel of that sharing knows the plain epilogues only), and with a
# few hundred rows the output and down projections are all left-over tiles: at 256 rows the down projection took
# 109 us handing over against 40 us shared (a prompt of 256 tokens 9.2 against 6.0 ms); the Llama-3.2-1B shape's
# projections (2,048 wide) fill the SMs only from 2,048 rows on.  Both can be set in the environment.
HANDOVER_MIN_ROWS = int(os.environ.get("STRATUM_HANDOVER_MIN_ROWS", 256))
HANDOVER_MIN_TILES = int(os.environ.get("STRATUM_HANDOVER_MIN_TILES", 60))


def hands_over(rows: int, out_features: int) -> bool:
    return (rows >= HANDOVER_MIN_ROWS
            and ((rows + 255) // 256) * ((out_features + 255) // 256) >= HANDOVER_MIN_TILES)


SKINNY_MAX_ROWS = int(os.environ.get("STRATUM_SKINNY_MAX_ROWS", 8))
STREAMK_MIN_WEIGHTS = int(os.environ.get("STRATUM_STREAMK_MIN_WEIGHTS", 20_000_000))


def _aligned(x: torch.Tensor, w: torch.Tensor) -> bool:
    k = w.shape[1]
    return (k % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def takes_tensor_cores(x: torch.Tensor, w: torch.Tensor, extras: bool) -> bool:
    """Whether this product goes to gemm_tc.  extras: the call carries work only gemm_tc's epilogues do (rows of
    a handed-over norm, the query/key/value epilogue), which decides where the weight-streaming kernel would
    otherwise have been taken."""
    if x.dtype != torch.bfloat16 or not _aligned(x, w):
        return False
    return extras or not (x.shape[0] <= SKINNY_MAX_ROWS and w.numel() < STREAMK_MIN_WEIGHTS)


def run(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, mode: int,
        extra=None) -> None:
    """out (=|+=) epilogue(x @ w.T + bias); see the EPI_* modes in kernels.py."""
    if extra is not None:
        if not takes_tensor_cores(x, w, extras=True):
            raise K.KernelError("this product carries epilogue work that only the tensor-core kernel does, and its "
                                "shape is not one that kernel takes")
        K.gemm_tc(x, w, bias, out, mode, extra)
        return
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
