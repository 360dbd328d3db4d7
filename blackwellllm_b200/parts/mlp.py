"""Dense gated feed-forward (SwiGLU): residual += W_down (silu(W_gate x) * W_up x).

Reference: src/core/engine.cpp:1010-1024 and src/kernels/swiglu.cu:15-37
(silu(g) = g / (1 + exp(-g))); no biases.  Gate and up are one matrix made at
load, so the input is read once.  On the bfloat16 tensor-core path their rows are
interleaved in blocks of 16 and the activation is computed in the epilogue of
that matrix product, so gate and up never travel through memory; otherwise (the
32-bit path, or sizes the tensor-core kernel refuses) the rows are gate then up
and a separate kernel applies the activation.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from .base import BuildContext, FeedForward, ParamSpec, register_ffn
from .linear import Linear


class SwiGLU(FeedForward):
    def __init__(self, spec, hidden_size: int, ctx: BuildContext):
        self.intermediate_size = int(spec.intermediate_size)
        self.hidden_size = hidden_size
        self.ctx = ctx
        self.fused = False
        self.gate_up: Linear = None
        self.down: Linear = None

    def param_specs(self) -> List[ParamSpec]:
        I, H = self.intermediate_size, self.hidden_size
        return [ParamSpec("gate_proj.weight", (I, H)), ParamSpec("up_proj.weight", (I, H)),
                ParamSpec("down_proj.weight", (H, I))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        self.fused = (g.dtype == torch.bfloat16 and g.is_cuda and self.intermediate_size % ops.SWIGLU_BLOCK == 0
                      and self.hidden_size % 8 == 0)
        if self.fused:
            self.gate_up = Linear(ops.interleave_gate_up(g, u))
        else:
            self.gate_up = Linear(torch.cat([g, u], dim=0))
        self.down = Linear(tensors["down_proj.weight"])

    def forward(self, x, residual, batch) -> None:
        if self.fused:
            a = ops.gemm_tc(x, self.gate_up.weight, swiglu=True)
        else:
            a = ops.swiglu(self.gate_up(x))
        self.down.add_to(a, residual)


register_ffn("swiglu", SwiGLU)
