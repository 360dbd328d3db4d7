"""Chooses one token per logits row on the device.

Per row: an optional repetition penalty on the tokens the request has emitted, then
greedy, or temperature softmax with an optional nucleus and an inverse CDF draw at a
uniform number that the host takes from the request's own Philox stream
(``sampling.params.uniform(seed, draw_index)``).  One small upload of (temperature,
top_p, u) per step (and one of the penalized ids where a request asks for the
penalty), one or two kernels, one read-back of the tokens.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..kernels import ops
from .params import SamplingParams, uniform


class Sampler:
    def __init__(self, device: torch.device):
        self.device = device

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               draw_index: Sequence[int], generated: Optional[Sequence[Sequence[int]]] = None) -> List[int]:
        """``logits`` [R, V] float32 on the device; row r uses params[r] and the
        ``draw_index[r]``-th number of the stream of ``seeds[r]``.  ``generated[r]``: what
        request r has emitted so far, for its repetition penalty (the logits are changed
        in place then)."""
        return self.sample_async(logits, params, seeds, draw_index, generated).tolist()

    def penalize(self, logits: torch.Tensor, params: Sequence[SamplingParams],
                 generated: Sequence[Sequence[int]]) -> None:
        """The repetition penalty of every row that asks for it, in place."""
        R = logits.shape[0]
        if len(generated) != R:
            raise ValueError("one history per logits row")
        acts = [list(p.penalized(g)) for p, g in zip(params, generated)]
        total = sum(len(a) for a in acts)
        if total == 0:
            return
        host = torch.empty((total + R + 1,), dtype=torch.int32, pin_memory=True)
        pen = torch.empty((R,), dtype=torch.float32, pin_memory=True)
        ids, begin = host.numpy(), [0]
        for a in acts:
            if a:
                ids[begin[-1]:begin[-1] + len(a)] = a
            begin.append(begin[-1] + len(a))
        ids[total:] = begin   # where each row's ids begin, and the end of the last
        pen.numpy()[:] = [p.repetition_penalty if a else 1.0 for p, a in zip(params, acts)]
        dev = host.to(self.device, non_blocking=True)
        ops.repetition_penalty(logits, dev[:total], dev[total:], pen.to(self.device, non_blocking=True))

    def sample_async(self, logits, params, seeds, draw_index, generated=None) -> torch.Tensor:
        R = logits.shape[0]
        if R != len(params):
            raise ValueError("one SamplingParams per logits row")
        if generated is not None:
            self.penalize(logits, params, generated)
        if all(p.greedy for p in params):
            return ops.sample(logits, None, None, None)
        host = torch.empty((3, R), dtype=torch.float32, pin_memory=True)
        rows = host.numpy()   # filled row by row: one assignment each instead of one per request
        rows[0] = [0.0 if p.greedy else p.temperature for p in params]
        rows[1] = [p.top_p for p in params]
        rows[2] = [0.0 if p.greedy else uniform(seeds[r], draw_index[r]) for r, p in enumerate(params)]
        dev = host.to(self.device, non_blocking=True)
        return ops.sample(logits, dev[0], dev[1], dev[2])
