"""Grouped-query softmax attention over paged keys and values.

In the reference's order (src/core/engine.cpp:968-990): q, k, v = W x (+ bias, added
once after the dot product and before the rotation, bf16_linear_bias.cu:44-50);
rotation of q and k; append of k and v to the cache; causal attention with
scale head_dim**-0.5 applied to the scores (paged_flash_attention.cu:142-144,446);
output projection added to the residual stream (bf16_linear_residual.cu:42-46).

Here the three projections are one matrix (rows q, k, v) made at load, its result
stays float32 until the rotation, and the residual sum is float32.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from .base import (BuildContext, Mixer, PagedKVRequest, ParamSpec, build_position, register_mixer)
from .linear import Linear


class GQAAttention(Mixer):
    def __init__(self, spec, hidden_size: int, ctx: BuildContext):
        self.nh, self.nkv, self.hd = int(spec.num_heads), int(spec.num_kv_heads), int(spec.head_dim)
        if self.nh % self.nkv:
            raise ValueError(f"num_heads {self.nh} is not a multiple of num_kv_heads {self.nkv}")
        self.hidden_size = hidden_size
        self.qkv_bias = bool(spec.qkv_bias)
        self.window = spec.window
        self.scale = float(spec.softmax_scale) if spec.softmax_scale is not None else self.hd ** -0.5
        self.ctx = ctx
        self.position = build_position(spec.position, self.hd, ctx)
        ops.check_attention_supported(ctx.dtype, self.hd, self.nh // self.nkv)
        self.qkv: Linear = None
        self.project = None
        self.o: Linear = None

    def cache_request(self):
        return PagedKVRequest(self.nkv, self.hd, self.window)

    def param_specs(self) -> List[ParamSpec]:
        H, q, kv = self.hidden_size, self.nh * self.hd, self.nkv * self.hd
        specs = [ParamSpec("q_proj.weight", (q, H)), ParamSpec("k_proj.weight", (kv, H)),
                 ParamSpec("v_proj.weight", (kv, H)), ParamSpec("o_proj.weight", (H, q))]
        if self.qkv_bias:
            specs += [ParamSpec("q_proj.bias", (q,), role="bias", init="bias_normal"),
                      ParamSpec("k_proj.bias", (kv,), role="bias", init="bias_normal"),
                      ParamSpec("v_proj.bias", (kv,), role="bias", init="bias_normal")]
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        w = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]], dim=0)
        b = None
        if self.qkv_bias:
            bs = [tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"]]
            dt = bs[0].dtype if all(t.dtype == bs[0].dtype for t in bs) else torch.float32
            b = torch.cat([t.to(dt) for t in bs], dim=0)
        # an encoding that runs inside the projection takes the weight over; else project, then encode
        self.project = self.position.fuse_projection(w, b, self.nh, self.nkv, self.hd)
        self.qkv = Linear(w, b) if self.project is None else None
        self.o = Linear(tensors["o_proj.weight"])

    def forward(self, x, residual, batch, cache, owns_cache: bool = True) -> None:
        if self.project is not None:
            q = self.project(x, batch, cache, owns_cache)
        else:
            qkv = self.qkv(x, out_dtype=torch.float32)
            q = self.position.rotate_append(qkv, batch, cache, self.nh, self.nkv, self.hd, append=owns_cache)
        o = ops.paged_attention(q, cache.k_pages, cache.v_pages, batch, batch.block_tables[cache.group],
                                self.nh, self.window, self.scale)
        self.o.add_to(o, residual)


register_mixer("gqa_attention", GQAAttention)
