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

STORE, ADD_TO_F32, STORE_F32, SWIGLU, QKV_ROPE = (K.EPI_STORE, K.EPI_ADD_F32, K.EPI_STORE_F32, K.EPI_SWIGLU,
                                                    K.EPI_QKV_ROPE)


class Linear:
    def __init__(self, runtime: Runtime, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        if weight.dim() != 2:
            raise ValueError("linear weight must be [out, in]")
        self.runtime = runtime
        self.weight = weight
        self.bias = bias
        self.out_features, self.in_features = weight.shape

    def __call__(self, x, out: Optional[torch.Tensor] = None, mode: int = STORE, emit=None, extra=None) -> torch.Tensor:
        """mode STORE: new tensor of x's dtype; ADD_TO_F32: out (float32) += y; STORE_F32: float32 out;
        SWIGLU: rows of W alternate gate and up, out[m][j] = silu(y[m][2j]) * y[m][2j+1] in x's dtype;
        QKV_ROPE: see kernels.GemmExtra (extra carries the cache and the rotation table; out: the query rows).
        x may be NormedRows (the product then applies the norm's row factors).  emit: a Handover that the
        ADD_TO_F32 product honours where it can (emit.result is then set)."""
        from . import gemm_dispatch
        from .base import NormedRows
        normed = x if isinstance(x, NormedRows) else None
        if normed is not None:
            x = normed.x
            extra = (extra or K.GemmExtra()).scaled_rows(normed.ss, normed.parts, normed.size, normed.eps)
        M = x.shape[0]
        if out is None:
            if mode == ADD_TO_F32:
                raise ValueError("ADD_TO_F32 needs the tensor to add into")
            width = self.out_features // 2 if mode == SWIGLU else self.out_features
            out = self.runtime.empty(M, width, dtype=torch.float32 if mode == STORE_F32 else x.dtype)
        if M == 0:
            return out
        if (emit is not None and mode == ADD_TO_F32 and gemm_dispatch.hands_over(M, self.out_features)
                and self.out_features % 128 == 0 and out.stride(0) % 4 == 0
                and gemm_dispatch.takes_tensor_cores(x, self.weight, extras=False)):
            xb = self.runtime.empty(M, self.out_features, dtype=torch.bfloat16)
            ss = self.runtime.empty(self.out_features // 128, M, dtype=torch.float32)
            extra = (extra or K.GemmExtra()).emit(xb, emit.gain, ss)
            parts = K.gemm_tc(x, self.weight, self.bias, out, K.EPI_ADD_F32_EMIT, extra)
            emit.result = NormedRows(xb, ss, parts, emit.size, emit.eps)
            return out
        gemm_dispatch.run(x, self.weight, self.bias, out, mode, extra)
        return out
