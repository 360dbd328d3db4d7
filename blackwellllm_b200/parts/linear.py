"""A weight matrix [out, in] with an optional bias, and the one place that picks
the matrix-product kernel for it.

float32 weights run on the CUDA cores with float32 FMAs (the true 32-bit path).
bfloat16 weights run on the tcgen05 tensor-core kernel; a shape that kernel
refuses (an inner size that is no multiple of 8, which a TMA row stride cannot
express) runs on the CUDA-core kernel with bfloat16 operands and float32 sums.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        if weight.dim() != 2:
            raise ValueError("Linear: weight must be [out, in]")
        self.weight = weight.contiguous()
        self.bias = None if bias is None else bias.contiguous()
        self.out_features, self.in_features = weight.shape

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None, accumulate: bool = False) -> torch.Tensor:
        """``out (=|+=) x @ W.T (+ bias)``.  ``accumulate`` adds into ``out`` (float32)."""
        w = self.weight
        if x.dtype != w.dtype:
            raise ops.KernelError(f"Linear: input is {x.dtype}, weight is {w.dtype}")
        if w.dtype == torch.bfloat16 and ops.gemm_tc_supports(x, w):
            return ops.gemm_tc(x, w, self.bias, out=out, out_dtype=out_dtype, accumulate=accumulate)
        return ops.gemm_simt(x, w, self.bias, out=out, out_dtype=out_dtype, accumulate=accumulate)

    def add_to(self, x: torch.Tensor, residual: torch.Tensor) -> None:
        """``residual += x @ W.T (+ bias)`` (float32).  For a few tokens on the tensor-core path the sum
        of the K splits is left to the next reader of ``residual`` (``ops.gemm_tc_deferred``)."""
        w = self.weight
        T = x.shape[0]
        if (ops.DEFER_SUMS and w.dtype == torch.bfloat16 and x.dtype == w.dtype and T <= ops.DEFER_MAX_TOKENS
                and T * w.shape[0] <= ops.PLANE_BUFFER_ELEMS and residual.dtype == torch.float32
                and residual.is_contiguous() and ops.gemm_tc_supports(x, w)):
            ops.gemm_tc_deferred(x, w, self.bias, residual)
        else:
            self(x, out=residual, accumulate=True)
