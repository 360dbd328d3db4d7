"""Typed descriptions of the parts a decoder is assembled from.

A model is data: a tuple of :class:`LayerSpec` (what each layer is made of) and a
tuple of :class:`ScheduleEntry` (the order in which layers run, and whose cache
each run reads).  Every size and constant lives in a spec; no part reads a
config.json key itself and no part knows which model it belongs to.

Each spec carries a ``kind`` string.  The part registries
(``blackwellllm_b200.parts.registry``) map ``kind`` to the class that builds the
part, so a new mixer, feed-forward, norm or position encoding is a new spec
dataclass plus one ``register_*`` call.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class Llama3RopeScaling:
    """Wavelength-band rescaling of rotary frequencies.

    Reference: src/kernels/rope.cuh:24-38 (apply_rope_scaling) and the keys read
    at src/core/config.cpp:263-273.
    """
    factor: float = 8.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192
    kind: str = "llama3"


@dataclass(frozen=True)
class RopeSpec:
    """rotate_half rotary position encoding over the first ``rotary_dim`` channels."""
    theta: float
    rotary_dim: int
    scaling: Optional[Llama3RopeScaling] = None
    kind: str = "rope"


@dataclass(frozen=True)
class NoPositionSpec:
    """A mixer that encodes no position (keys and queries are used as projected)."""
    kind: str = "none"


@dataclass(frozen=True)
class RMSNormSpec:
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query softmax attention over a paged key/value cache.

    ``window`` is the number of most recent keys (the query's own position
    included) a query may see; ``None`` means all of them.
    """
    num_heads: int
    num_kv_heads: int
    head_dim: int
    qkv_bias: bool
    position: Any  # RopeSpec | NoPositionSpec | any registered position spec
    window: Optional[int] = None
    softmax_scale: Optional[float] = None  # None -> head_dim ** -0.5
    kind: str = "gqa_attention"


@dataclass(frozen=True)
class SwiGLUSpec:
    """Dense gated feed-forward: down(silu(gate(x)) * up(x))."""
    intermediate_size: int
    kind: str = "swiglu"


@dataclass(frozen=True)
class LayerSpec:
    """One layer: which mixer, which feed-forward, which norms, arranged how.

    ``block`` names the arrangement (``"prenorm"``: x += mixer(norm(x));
    x += ffn(norm(x))).  ``ffn`` may be ``None`` for a mixer-only layer.
    """
    mixer: Any
    ffn: Any
    mixer_norm: Any
    ffn_norm: Any
    block: str = "prenorm"
    # where each part's tensors sit below the layer's prefix in the checkpoint
    mixer_prefix: str = "self_attn."
    ffn_prefix: str = "mlp."
    mixer_norm_prefix: str = "input_layernorm."
    ffn_norm_prefix: str = "post_attention_layernorm."


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``cache_of`` is the schedule position whose cache this
    run reads instead of owning one (``None``: it owns its cache and appends to it).
    A layer index may appear in several entries (weights shared, caches separate).
    """
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelConfig:
    """Everything the engine needs to know about one checkpoint's architecture."""
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: Any
    tie_word_embeddings: bool
    max_position_embeddings: int  # 0 = not stated
    weight_prefix: str = "model."
    layer_prefix: str = "model.layers.{i}."
    embed_name: str = "model.embed_tokens.weight"
    final_norm_prefix: str = "model.norm."
    head_name: str = "lm_head.weight"
    # what a decoder may do besides its blocks (all off by default): the embedding rows times a
    # constant, the logits times a constant, and a soft cap  cap * tanh(logits / cap)
    embedding_multiplier: float = 1.0
    logit_scale: float = 1.0
    logit_softcap: Optional[float] = None
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    stored_dtype: str = "bfloat16"
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, hash=False)

    @property
    def num_layers(self) -> int:
        return len(self.layers)
