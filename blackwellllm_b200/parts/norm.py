"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, the sum and the scaling in float32.

Formula of the reference: src/kernels/rmsnorm.cu:107-120,133-138 (it sums in
double and rounds twice through bfloat16; here: one float32 computation and one
rounding on store).  ``rows`` normalises only the named rows (final norm on the
positions whose logits are wanted, src/core/engine.cpp:1029-1035).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import BuildContext, Norm, ParamSpec, register_norm


class RMSNorm(Norm):
    adds_pending = True

    def __init__(self, spec, hidden_size: int, ctx: BuildContext):
        self.eps = float(spec.eps)
        self.hidden_size = hidden_size
        self.ctx = ctx
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec("weight", (self.hidden_size,), role="gain", init="ones")]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, self.ctx.dtype, rows=rows)


register_norm("rmsnorm", RMSNorm)
