"""Interfaces of the parts a decoder is put together from, and their registries.

A part is built from its spec (``config.specs``) and the model's hidden size, says
which tensors it wants (:meth:`Part.param_specs`), receives them
(:meth:`Part.bind`) and then runs on the step's batch.  No part knows which model
it is in: sizes and constants come from the spec alone.

Interfaces
----------
Norm            ``forward(x_f32[T,H], rows=None) -> [n,H]`` in the compute dtype.
PositionEncoding ``rotate_append(qkv, batch, cache, nh, nkv, hd) -> q``: encodes the
                position into queries and keys and appends keys and values to
                the cache pages of the tokens' positions.
Mixer           ``cache_request()`` says what cache it needs (paged keys/values,
                a fixed-size state per request, or nothing);
                ``forward(x, residual, batch, cache, owns_cache)`` adds its output
                to ``residual`` (float32 [T,H]) in place; ``owns_cache`` is false
                when this run reads the cache of another run and must not write it.
FeedForward     ``forward(x, residual, batch)`` adds its output to ``residual``.
Block           ``forward(residual, batch, cache)`` arranges norms, mixer and
                feed-forward.

Registering: ``register_mixer("kind", Class)`` (and ``register_ffn``,
``register_norm``, ``register_position``, ``register_block``); ``Class(spec,
hidden_size, ctx)`` builds it.  The spec is any object with a ``kind`` attribute.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch


@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part wants, named relative to the part's prefix.

    role: ``"matrix"`` (operand of a matrix product or an embedding table: held in
    the compute dtype), ``"gain"`` / ``"bias"`` (vectors: a 32-bit stored tensor
    stays 32-bit), ``"int_table"`` (held as int32).  ``init``: how the
    random-weights mode fills it (``"normal"``, ``"ones"``, ``"bias_normal"``,
    ``"zeros"``).
    """
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    optional: bool = False


@dataclass(frozen=True)
class BuildContext:
    device: torch.device
    dtype: torch.dtype  # torch.float32 (true 32-bit path) or torch.bfloat16


@dataclass(frozen=True)
class PagedKVRequest:
    """A mixer's need for paged keys and values: per token ``2 * num_kv_heads *
    head_dim`` elements; ``window``: only that many latest tokens stay needed."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class FixedStateRequest:
    """A mixer's need for a state of fixed size per request (zeroed at admission)."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    def param_specs(self) -> List[ParamSpec]:
        return []

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receives the tensors named by :meth:`param_specs` (device, final dtype)."""


class Norm(Part):
    # True: forward() reads x only through ops.rmsnorm, which adds a sum that a matrix product left
    # outstanding for x (ops.gemm_tc_deferred) while it normalises.  False: whoever calls forward()
    # calls ops.resolve_pending() first.
    adds_pending = False

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def rotate_append(self, qkv, batch, cache, nh: int, nkv: int, hd: int, append: bool = True) -> torch.Tensor:
        """qkv [T, (nh + 2 nkv) * hd] float32 -> encoded queries [T, nh * hd]; encoded keys and raw
        values are written to the cache when ``append``."""
        raise NotImplementedError

    def fuse_projection(self, weight: torch.Tensor, bias: Optional[torch.Tensor], nh: int, nkv: int, hd: int):
        """Optional: an encoding that can run inside the q/k/v projection returns a callable
        ``project(x, batch, cache, append) -> queries`` that replaces projection plus
        :meth:`rotate_append` (it may keep its own copy of ``weight`` and ``bias`` in another
        row order).  None: the mixer projects and calls :meth:`rotate_append`."""
        return None


class Mixer(Part):
    graph_safe = True  # False: forward() does host work between kernels; decode steps then run uncaptured

    def cache_request(self):
        return None

    def forward(self, x, residual, batch, cache, owns_cache: bool = True) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, residual, batch) -> None:
        raise NotImplementedError


class Block(Part):
    mixer: Mixer
    # True: forward() may be entered, and may return, with a sum outstanding for the residual stream
    # (ops.gemm_tc_deferred) and sees to it that no part reads the stream before the sum is made.
    takes_pending = False

    def forward(self, residual, batch, cache, owns_cache: bool = True) -> None:
        raise NotImplementedError


_REG: Dict[str, Dict[str, Callable[..., Any]]] = {
    "mixer": {}, "ffn": {}, "norm": {}, "position": {}, "block": {}}


def _register(family: str, kind: str, cls) -> None:
    _REG[family][kind] = cls


def register_mixer(kind: str, cls): _register("mixer", kind, cls)
def register_ffn(kind: str, cls): _register("ffn", kind, cls)
def register_norm(kind: str, cls): _register("norm", kind, cls)
def register_position(kind: str, cls): _register("position", kind, cls)
def register_block(kind: str, cls): _register("block", kind, cls)


def _build(family: str, spec, *args):
    kind = getattr(spec, "kind", None)
    table = _REG[family]
    if kind not in table:
        raise KeyError(f"no {family} registered for kind {kind!r}; registered: {sorted(table)}")
    return table[kind](spec, *args)


def build_mixer(spec, hidden_size: int, ctx: BuildContext) -> Mixer:
    return _build("mixer", spec, hidden_size, ctx)


def build_ffn(spec, hidden_size: int, ctx: BuildContext) -> FeedForward:
    return _build("ffn", spec, hidden_size, ctx)


def build_norm(spec, hidden_size: int, ctx: BuildContext) -> Norm:
    return _build("norm", spec, hidden_size, ctx)


def build_position(spec, head_dim: int, ctx: BuildContext) -> PositionEncoding:
    return _build("position", spec, head_dim, ctx)


def build_block(layer_spec, hidden_size: int, ctx: BuildContext) -> Block:
    table = _REG["block"]
    if layer_spec.block not in table:
        raise KeyError(f"no block registered for arrangement {layer_spec.block!r}; registered: {sorted(table)}")
    return table[layer_spec.block](layer_spec, hidden_size, ctx)
