"""Sampling parameters and the per-request random stream.

The reference samples with a temperature and a nucleus (top_p), greedy when the
temperature is (near) zero (src/kernels/sampling.cu:128-210), with defaults
temperature 0.6 and top_p 0.9 (include/blackwell/runtime_config.h:87-137;
scripts/cli_chat.py:77-85, which also caps a reply at 1024 new tokens).  Its
random source is an unseeded process-wide generator; here every request has its
own counter-based stream (Philox 4x32-10 keyed by the request's seed), so a
request's tokens do not depend on what else is in the batch.  The reference's
repetition penalty (src/kernels/sampling.cuh:10-29: each distinct id of a rolling
window of emitted tokens has its logit divided by the penalty when positive and
multiplied when not, before temperature, nucleus or argmax) is a parameter too.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

_M0, _M1 = 0xD2511F53, 0xCD9E8D57
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_MASK = 0xFFFFFFFF


def philox4x32(counter: Tuple[int, int, int, int], key: Tuple[int, int]) -> Tuple[int, int, int, int]:
    c0, c1, c2, c3 = counter
    k0, k1 = key
    for _ in range(10):
        p0 = _M0 * c0
        p1 = _M1 * c2
        c0, c1, c2, c3 = ((p1 >> 32) ^ c1 ^ k0) & _MASK, p1 & _MASK, ((p0 >> 32) ^ c3 ^ k1) & _MASK, p0 & _MASK
        k0 = (k0 + _W0) & _MASK
        k1 = (k1 + _W1) & _MASK
    return c0, c1, c2, c3


def uniform(seed: int, index: int) -> float:
    """The ``index``-th number of the stream of ``seed``: uniform in [0, 1) with 24 bits."""
    r = philox4x32((index & _MASK, (index >> 32) & _MASK, 0, 0), (seed & _MASK, (seed >> 32) & _MASK))
    return (r[0] >> 8) * (1.0 / (1 << 24))


@dataclass
class SamplingParams:
    """temperature 0 is greedy (lowest index wins a tie).  ``top_p`` < 1 keeps the
    most probable tokens whose mass reaches it.  ``seed`` None: derived from the
    engine's seed and the request's number.  ``repetition_penalty`` > 1 makes the
    request's last ``repetition_window`` generated tokens (0: all of them) less
    likely; <= 1 is off."""
    temperature: float = 0.6
    top_p: float = 0.9
    max_new_tokens: int = 1024
    seed: Optional[int] = None
    stop_token_ids: Tuple[int, ...] = ()
    ignore_eos: bool = False
    repetition_penalty: float = 1.0
    repetition_window: int = 64

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if not 0 < self.top_p <= 1:
            raise ValueError("top_p must be in (0, 1]")
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be >= 1")
        if not self.repetition_penalty > 0:
            raise ValueError("repetition_penalty must be > 0 (<= 1 switches it off)")
        if self.repetition_window < 0:
            raise ValueError("repetition_window must be >= 0")

    def penalized(self, generated: Sequence[int]) -> Sequence[int]:
        """The ids that the repetition penalty acts on, given what the request has generated."""
        if not self.repetition_penalty > 1.0 or not generated:
            return ()
        return generated[-self.repetition_window:] if self.repetition_window else generated

    @property
    def greedy(self) -> bool:
        return self.temperature < 1e-5  # the reference's threshold, sampling.cu:130
