"""Position encodings for attention mixers.

:class:`RotaryEncoding` is rotate_half RoPE (src/kernels/rope.cu:7-35): pair
(j, j + rd/2) of each query and key head turns by ``pos * inv_freq[j]``,
``inv_freq[j] = theta ** (-2j/rd)``, optionally rescaled by the llama3
wavelength bands (src/kernels/rope.cuh:24-38).  The table is computed once on the
host in float64 and stored as float32; the angle is the float32 product
``float(pos) * inv_freq[j]`` and sine/cosine are the precise ones.

:class:`NoPosition` rotates nothing.  Both append rotated keys and raw values to
the cache pages in the same kernel.
"""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from .base import BuildContext, PositionEncoding, register_position


def rotary_inv_freq(theta: float, rotary_dim: int, scaling=None) -> torch.Tensor:
    j = torch.arange(rotary_dim // 2, dtype=torch.float64)
    inv = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * j / rotary_dim)
    if scaling is not None:
        if getattr(scaling, "kind", None) != "llama3":
            raise ValueError(f"unknown rope scaling {scaling!r}")
        orig = float(scaling.original_max_position_embeddings)
        low, high, factor = scaling.low_freq_factor, scaling.high_freq_factor, scaling.factor
        wavelen = 2.0 * math.pi / inv
        smooth = (orig / wavelen - low) / (high - low)
        mid = (1.0 - smooth) * inv / factor + smooth * inv
        inv = torch.where(wavelen < orig / high, inv,
                          torch.where(wavelen > orig / low, inv / factor, mid))
    return inv.to(torch.float32)


class RotaryEncoding(PositionEncoding):
    def __init__(self, spec, head_dim: int, ctx: BuildContext):
        if spec.rotary_dim % 2 or not 0 < spec.rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even and in (0, head_dim={head_dim}]")
        self.rotary_dim = int(spec.rotary_dim)
        self.inv_freq = rotary_inv_freq(spec.theta, self.rotary_dim, spec.scaling).to(ctx.device)
        self._key = ("rope_table", float(spec.theta), self.rotary_dim, spec.scaling)

    def _table(self, batch):
        # the cosines and sines of the step's positions are the same in every layer with these
        # rotary parameters: computed by the first one, kept on the batch for the others
        table = batch.extras.get(self._key)
        if table is None:
            table = ops.rope_table(batch.positions, self.inv_freq, self.rotary_dim)
            batch.extras[self._key] = table
        return table

    def rotate_append(self, qkv, batch, cache, nh, nkv, hd, append=True):
        table = self._table(batch)
        return ops.rope_append(qkv, batch.positions, batch.req_of_token, batch.block_tables[cache.group],
                               self.inv_freq, self.rotary_dim, cache.k_pages, cache.v_pages, nh, nkv, hd,
                               append=append, table=table)


    def fuse_projection(self, weight, bias, nh, nkv, hd):
        # bfloat16 on the tensor-core product: rotation and append run in its epilogue
        if weight.dtype != torch.bfloat16 or not weight.is_cuda or weight.shape[1] % 8:
            return None
        order = ops.rotary_row_order(nh, nkv, hd, self.rotary_dim).to(weight.device)
        w = weight.index_select(0, order).contiguous()
        b = bias.index_select(0, order).contiguous() if bias is not None else None

        def project(x, batch, cache, append=True):
            if batch.T <= ops.GEMM_FUSED_REDUCE_MAX_TOKENS:
                # few tokens: the product leaves its K splits as planes, which the rotation's kernel
                # adds while it reads them (the rotation in the product's own epilogue, after a sum
                # of the splits in its last warps, was measured slower than a kernel of its own)
                qkv = ops.gemm_tc_planes(x, w, b) if ops.DEFER_SUMS else ops.gemm_tc(x, w, b, out_dtype=torch.float32)
                table = self._table(batch)

                def rotate():
                    return ops.rope_append(qkv, batch.positions, batch.req_of_token, batch.block_tables[cache.group],
                                           self.inv_freq, self.rotary_dim, cache.k_pages, cache.v_pages, nh, nkv, hd,
                                           append=append, table=table, paired=True)
                if (qkv.dim() == 3 and batch.T == batch.R
                        and ops.attention_takes_unrotated(hd, cache.k_pages.shape[2])):
                    # one token per request: the attention's key-slice kernel rotates and appends by itself
                    return ops.UnrotatedQKV(qkv, table, self.rotary_dim, append, rotate)
                return rotate()
            slots = None
            if append:   # where the step's tokens go in this cache group: the same for all its layers
                key = ("kv_slots", cache.group)
                slots = batch.extras.get(key)
                if slots is None:
                    slots = ops.kv_slots(batch.positions, batch.req_of_token, batch.block_tables[cache.group],
                                         cache.k_pages.shape[2], cache.k_pages.shape[0])
                    batch.extras[key] = slots
            return ops.gemm_tc_rope(x, w, b, self._table(batch), slots, cache.k_pages, cache.v_pages, nh, nkv, hd,
                                    self.rotary_dim)
        return project


class NoPosition(PositionEncoding):
    def __init__(self, spec, head_dim: int, ctx: BuildContext):
        pass

    def rotate_append(self, qkv, batch, cache, nh, nkv, hd, append=True):
        return ops.rope_append(qkv, batch.positions, batch.req_of_token, batch.block_tables[cache.group],
                               None, 0, cache.k_pages, cache.v_pages, nh, nkv, hd, append=append)


register_position("rope", RotaryEncoding)
register_position("none", NoPosition)
