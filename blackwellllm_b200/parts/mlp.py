"""Dense gated feed-forward (SwiGLU): residual += W_down (silu(W_gate x) * W_up x).

Reference: src/core/engine.cpp:1010-1024 and src/kernels/swiglu.cu:15-37
(silu(g) = g / (1 + exp(-g))); no biases.  Gate and up are one matrix made at
load (rows gate, then up), so the input is read once.
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
        self.gate_up: Linear = None
        self.down: Linear = None

    def param_specs(self) -> List[ParamSpec]:
        I, H = self.intermediate_size, self.hidden_size
        return [ParamSpec("gate_proj.weight", (I, H)), ParamSpec("up_proj.weight", (I, H)),
                ParamSpec("down_proj.weight", (H, I))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.gate_up = Linear(torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], dim=0))
        self.down = Linear(tensors["down_proj.weight"])

    def forward(self, x, residual, batch) -> None:
        gu = self.gate_up(x)
        a = ops.swiglu(gu)
        self.down(a, out=residual, accumulate=True)


register_ffn("swiglu", SwiGLU)
