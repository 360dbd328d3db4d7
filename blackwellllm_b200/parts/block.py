"""Arrangements of norms, mixer and feed-forward in a layer.

``prenorm`` (src/core/engine.cpp:946-1024): the norm stands before each sublayer
and reads the residual stream without changing it; each sublayer adds its output
to the residual stream, which stays float32.  A sublayer's last product may leave its sum to the
next reader of the stream (``Linear.add_to``): the next norm, which adds it while it normalises.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from .base import (Block, BuildContext, ParamSpec, build_ffn, build_mixer, build_norm,
                   register_block)


class PreNormBlock(Block):
    def __init__(self, layer_spec, hidden_size: int, ctx: BuildContext):
        self.spec = layer_spec
        self.mixer_norm = build_norm(layer_spec.mixer_norm, hidden_size, ctx)
        self.mixer = build_mixer(layer_spec.mixer, hidden_size, ctx)
        self.ffn = None
        self.ffn_norm = None
        if layer_spec.ffn is not None:
            self.ffn_norm = build_norm(layer_spec.ffn_norm, hidden_size, ctx)
            self.ffn = build_ffn(layer_spec.ffn, hidden_size, ctx)

    def _children(self):
        s = self.spec
        kids = [(s.mixer_norm_prefix, self.mixer_norm), (s.mixer_prefix, self.mixer)]
        if self.ffn is not None:
            kids += [(s.ffn_norm_prefix, self.ffn_norm), (s.ffn_prefix, self.ffn)]
        return kids

    def param_specs(self) -> List[ParamSpec]:
        out = []
        for prefix, part in self._children():
            for p in part.param_specs():
                out.append(ParamSpec(prefix + p.name, p.shape, p.role, p.init, p.optional))
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for prefix, part in self._children():
            part.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)})

    takes_pending = True

    @staticmethod
    def _normed(norm, residual):
        # a sublayer may have left the sum of its last product to the stream's next reader: a norm
        # that adds it while it normalises, or else a kernel of its own here
        if not norm.adds_pending:
            ops.resolve_pending()
        return norm.forward(residual)

    def forward(self, residual, batch, cache, owns_cache: bool = True) -> None:
        x = self._normed(self.mixer_norm, residual)
        self.mixer.forward(x, residual, batch, cache, owns_cache)
        if self.ffn is not None:
            x = self._normed(self.ffn_norm, residual)
            self.ffn.forward(x, residual, batch)


register_block("prenorm", PreNormBlock)
