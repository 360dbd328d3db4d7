"""The decoder that every registered architecture is run by: an embedding, blocks
built from the configuration's layer specs, a schedule that says in which order
they run and whose cache each run uses, a final norm and the output head; around
them the configuration's optional constants (embedding multiplier, logit scale,
logit soft cap).

It is driven by :class:`ModelConfig` alone and knows no architecture by name.
Reference for the sequence of operations: src/core/engine.cpp:921-1041.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.specs import ModelConfig
from ..kernels import ops
from ..parts import BuildContext, ParamSpec, build_block, build_norm
from ..parts.linear import Linear


class DecoderModel:
    def __init__(self, config: ModelConfig, ctx: BuildContext):
        self.config = config
        self.ctx = ctx
        H = config.hidden_size
        self.blocks = [build_block(ls, H, ctx) for ls in config.layers]
        self.final_norm = build_norm(config.final_norm, H, ctx)
        for e in config.schedule:
            if not 0 <= e.layer < len(self.blocks):
                raise ValueError(f"schedule names layer {e.layer}, the model has {len(self.blocks)}")
        for pos, e in enumerate(config.schedule):
            if e.cache_of is not None:
                if not 0 <= e.cache_of < pos or config.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {pos}: cache_of must name an earlier entry that owns its cache")
        self.embed: Optional[torch.Tensor] = None
        self.head: Optional[Linear] = None

    # ------------------------------------------------------------ parameters
    def param_specs(self) -> Dict[str, ParamSpec]:
        c = self.config
        specs: Dict[str, ParamSpec] = {}
        specs[c.embed_name] = ParamSpec(c.embed_name, (c.vocab_size, c.hidden_size))
        for i, blk in enumerate(self.blocks):
            prefix = c.layer_prefix.format(i=i)
            for p in blk.param_specs():
                specs[prefix + p.name] = ParamSpec(prefix + p.name, p.shape, p.role, p.init, p.optional)
        for p in self.final_norm.param_specs():
            name = c.final_norm_prefix + p.name
            specs[name] = ParamSpec(name, p.shape, p.role, p.init, p.optional)
        # a tied head reuses the embedding table; a stored lm_head is then tolerated and ignored
        specs[c.head_name] = ParamSpec(c.head_name, (c.vocab_size, c.hidden_size),
                                       optional=c.tie_word_embeddings)
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        c = self.config
        self.embed = tensors[c.embed_name].contiguous()
        for i, blk in enumerate(self.blocks):
            prefix = c.layer_prefix.format(i=i)
            blk.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)})
        stem = c.final_norm_prefix
        self.final_norm.bind({k[len(stem):]: v for k, v in tensors.items() if k.startswith(stem)})
        self.head = Linear(self.embed if c.tie_word_embeddings else tensors[c.head_name])

    # ------------------------------------------------------------ caches
    def cache_requests(self) -> List[object]:
        """Per schedule entry: what cache that run owns (None if it owns none)."""
        out = []
        for e in self.config.schedule:
            out.append(None if e.cache_of is not None else self.blocks[e.layer].mixer.cache_request())
        return out

    # ------------------------------------------------------------ forward
    def forward(self, batch, caches: List[object]) -> torch.Tensor:
        """Runs the batch's tokens through the schedule; returns float32 logits
        [len(batch.logit_rows), vocab] for the rows that were asked for."""
        c = self.config
        ops.discard_pending()   # nothing of an earlier (failed) pass is added into this one's tensors
        h = ops.embed_gather(self.embed, batch.token_ids, scale=c.embedding_multiplier)
        for pos, e in enumerate(self.config.schedule):
            cache = caches[e.cache_of if e.cache_of is not None else pos]
            blk = self.blocks[e.layer]
            if not blk.takes_pending:
                ops.resolve_pending()   # the block before may have left its last sum to the next reader
            blk.forward(h, batch, cache, owns_cache=e.cache_of is None)
        n = batch.logit_rows.numel()
        if n == 0:
            ops.discard_pending(h)
            return torch.empty((0, self.config.vocab_size), dtype=torch.float32, device=h.device)
        if not self.final_norm.adds_pending:
            ops.resolve_pending()
        x = self.final_norm.forward(h, rows=batch.logit_rows)
        ops.discard_pending(h)          # the stream ends here: only the chosen rows were summed
        logits = self.head(x, out_dtype=torch.float32)
        if c.logit_scale != 1.0 or c.logit_softcap is not None:
            ops.logit_transform(logits, c.logit_scale, c.logit_softcap)
        return logits
