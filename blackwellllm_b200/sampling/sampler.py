"""Chooses one token per logits row on the device.

Per row: greedy, or temperature softmax with an optional nucleus and an inverse
CDF draw at a uniform number that the host takes from the request's own Philox
stream (``sampling.params.uniform(seed, draw_index)``).  One small upload of
(temperature, top_p, u) per step, one kernel, one read-back of the tokens.
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from ..kernels import ops
from .params import SamplingParams, uniform


class Sampler:
    def __init__(self, device: torch.device):
        self.device = device

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               draw_index: Sequence[int]) -> List[int]:
        """``logits`` [R, V] float32 on the device; row r uses params[r] and the
        ``draw_index[r]``-th number of the stream of ``seeds[r]``."""
        return self.sample_async(logits, params, seeds, draw_index).tolist()

    def sample_async(self, logits, params, seeds, draw_index) -> torch.Tensor:
        R = logits.shape[0]
        if R != len(params):
            raise ValueError("one SamplingParams per logits row")
        if all(p.greedy for p in params):
            return ops.sample(logits, None, None, None)
        host = torch.empty((3, R), dtype=torch.float32, pin_memory=True)
        for r, p in enumerate(params):
            host[0, r] = 0.0 if p.greedy else p.temperature
            host[1, r] = p.top_p
            host[2, r] = 0.0 if p.greedy else uniform(seeds[r], draw_index[r])
        dev = host.to(self.device, non_blocking=True)
        return ops.sample(logits, dev[0], dev[1], dev[2])
