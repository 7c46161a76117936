"""y = x W^T + b: the one place that chooses a matrix-product kernel.

W is [out, in] row-major as stored in the file (stratum/native/stratum_linear.h:491-507).
float32: the CUDA-core kernel with a fixed summation order, always (the true 32-bit
path has no tensor-core mode).  bfloat16: the tensor-core kernels when the shape meets
their alignment rules, else the same CUDA-core kernel.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K
from .base import Runtime

STORE, ADD_TO_F32, STORE_F32, SWIGLU = K.EPI_STORE, K.EPI_ADD_F32, K.EPI_STORE_F32, K.EPI_SWIGLU


class Linear:
    def __init__(self, runtime: Runtime, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        if weight.dim() != 2:
            raise ValueError("linear weight must be [out, in]")
        self.runtime = runtime
        self.weight = weight
        self.bias = bias
        self.out_features, self.in_features = weight.shape

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, mode: int = STORE) -> torch.Tensor:
        """mode STORE: new tensor of x's dtype; ADD_TO_F32: out (float32) += y; STORE_F32: float32 out;
        SWIGLU: rows of W alternate gate and up, out[m][j] = silu(y[m][2j]) * y[m][2j+1] in x's dtype."""
        M = x.shape[0]
        if out is None:
            if mode == ADD_TO_F32:
                raise ValueError("ADD_TO_F32 needs the tensor to add into")
            width = self.out_features // 2 if mode == SWIGLU else self.out_features
            out = self.runtime.empty(M, width, dtype=torch.float32 if mode == STORE_F32 else x.dtype)
        if M == 0:
            return out
        from . import gemm_dispatch
        gemm_dispatch.run(x, self.weight, self.bias, out, mode)
        return out
