"""Llama / Qwen2 dense decoder: config.json -> :class:`ModelConfig`.

The architecture, as the reference runs it (src/core/engine.cpp:842-876):
embedding; per layer ``x += o(attn(rope(q(n1(x))), rope(k(n1(x))), v(n1(x))))``
then ``x += down(silu(gate(n2(x))) * up(n2(x)))``; final RMSNorm; lm_head.
Keys and defaults follow src/core/config.cpp:113-284:

* required: hidden_size, num_attention_heads, intermediate_size,
  num_hidden_layers, num_key_value_heads, vocab_size (config.cpp:126-131);
* head_dim defaults to hidden_size // num_attention_heads (config.cpp:144-145);
* rms_norm_eps (or its alias layernorm_epsilon) defaults to 1e-6 (config.cpp:157); rope_theta to
  10000 (config.cpp:188);
* q/k/v bias: ``attention_bias`` if present, else true exactly for model_type
  "qwen2" (config.cpp:226-227);
* tie_word_embeddings defaults to false (config.cpp:158);
* rope_scaling: only rope_type "llama3" (config.cpp:263-273).  The reference
  warns and carries on for other types; here that is an error, since the angles
  would be wrong;
* use_sliding_window=true is rejected (config.cpp:282-284), and so is a
  quantization_config (quantized weights are not handled by this engine).

This module only describes the model.  It builds nothing and owns no tensor.
"""
from __future__ import annotations

from typing import Any, Mapping

from ..config.registry import ConfigError, register_architecture
from ..config.specs import (AttentionSpec, LayerSpec, Llama3RopeScaling, ModelConfig,
                            RMSNormSpec, RopeSpec, ScheduleEntry, SwiGLUSpec)

_REQUIRED = ("hidden_size", "num_attention_heads", "intermediate_size",
             "num_hidden_layers", "num_key_value_heads", "vocab_size")


def _positive_int(raw: Mapping[str, Any], key: str) -> int:
    v = raw[key]
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {key!r} must be a positive integer, got {v!r}")
    return v


def _rope_scaling(raw: Mapping[str, Any]):
    rs = raw.get("rope_scaling")
    if rs is None:
        return None
    if not isinstance(rs, dict):
        raise ConfigError("config.json: 'rope_scaling' must be an object or null")
    rope_type = rs.get("rope_type", rs.get("type", "unknown"))
    if rope_type == "default":
        return None
    if rope_type != "llama3":
        raise ConfigError(
            f"config.json: rope_scaling type {rope_type!r} is not supported (only 'llama3')")
    factor = float(rs.get("factor", 8.0))
    low = float(rs.get("low_freq_factor", 1.0))
    high = float(rs.get("high_freq_factor", 4.0))
    orig = int(rs.get("original_max_position_embeddings", 8192))
    if factor <= 0 or orig <= 0 or high == low:
        raise ConfigError("config.json: rope_scaling needs factor > 0, "
                          "original_max_position_embeddings > 0 and high_freq_factor != low_freq_factor")
    return Llama3RopeScaling(factor=factor, low_freq_factor=low, high_freq_factor=high,
                             original_max_position_embeddings=orig)


def parse_dense_decoder(raw: Mapping[str, Any], *, architecture: str,
                        default_qkv_bias: bool) -> ModelConfig:
    missing = [k for k in _REQUIRED if k not in raw]
    if missing:
        raise ConfigError(f"config.json is missing required key(s): {missing}")
    hidden = _positive_int(raw, "hidden_size")
    heads = _positive_int(raw, "num_attention_heads")
    kv_heads = _positive_int(raw, "num_key_value_heads")
    inter = _positive_int(raw, "intermediate_size")
    n_layers = _positive_int(raw, "num_hidden_layers")
    vocab = _positive_int(raw, "vocab_size")
    if heads % kv_heads != 0:
        raise ConfigError(f"num_attention_heads ({heads}) is not a multiple of "
                          f"num_key_value_heads ({kv_heads})")
    if "head_dim" in raw and raw["head_dim"] is not None:
        head_dim = _positive_int(raw, "head_dim")
    else:
        if hidden % heads != 0:
            raise ConfigError(f"hidden_size ({hidden}) is not a multiple of num_attention_heads "
                              f"({heads}) and no head_dim is given")
        head_dim = hidden // heads
    if raw.get("use_sliding_window", False):
        raise ConfigError("use_sliding_window=true is not supported for this architecture")
    if "quantization_config" in raw:
        raise ConfigError("quantization_config present: quantized checkpoints are not supported")
    act = raw.get("hidden_act", "silu")
    if act != "silu":
        raise ConfigError(f"hidden_act {act!r} is not supported (the feed-forward is SwiGLU: 'silu')")
    eps = float(raw.get("rms_norm_eps", raw.get("layernorm_epsilon", 1e-6)))   # the alias: config.cpp:157
    if not eps > 0:
        raise ConfigError(f"rms_norm_eps must be > 0, got {eps!r}")
    theta = float(raw.get("rope_theta", 10000.0))
    if not theta > 0:
        raise ConfigError(f"rope_theta must be > 0, got {theta!r}")
    prf = float(raw.get("partial_rotary_factor", 1.0))
    rotary_dim = int(head_dim * prf)
    if rotary_dim <= 0 or rotary_dim > head_dim:
        rotary_dim = head_dim
    rotary_dim &= ~1
    if rotary_dim == 0:
        raise ConfigError("partial_rotary_factor leaves fewer than 2 rotated channels")
    model_type = raw.get("model_type", "")
    if "attention_bias" in raw:
        qkv_bias = bool(raw["attention_bias"])
    else:
        qkv_bias = (model_type == "qwen2") if model_type else default_qkv_bias
    tie = bool(raw.get("tie_word_embeddings", False))
    max_pos = int(raw.get("max_position_embeddings", 0) or 0)

    eos = raw.get("eos_token_id")
    if eos is None:
        eos_ids = ()
    elif isinstance(eos, int):
        eos_ids = (eos,)
    else:
        eos_ids = tuple(int(e) for e in eos)
    bos = raw.get("bos_token_id")

    rope = RopeSpec(theta=theta, rotary_dim=rotary_dim, scaling=_rope_scaling(raw))
    layer = LayerSpec(
        mixer=AttentionSpec(num_heads=heads, num_kv_heads=kv_heads, head_dim=head_dim,
                            qkv_bias=qkv_bias, position=rope, window=None),
        ffn=SwiGLUSpec(intermediate_size=inter),
        mixer_norm=RMSNormSpec(eps=eps),
        ffn_norm=RMSNormSpec(eps=eps),
        block="prenorm",
    )
    stored = str(raw.get("torch_dtype", raw.get("dtype", "bfloat16")))
    return ModelConfig(
        architecture=architecture,
        hidden_size=hidden,
        vocab_size=vocab,
        layers=tuple(layer for _ in range(n_layers)),
        schedule=tuple(ScheduleEntry(layer=i) for i in range(n_layers)),
        final_norm=RMSNormSpec(eps=eps),
        tie_word_embeddings=tie,
        max_position_embeddings=max_pos,
        eos_token_ids=eos_ids,
        bos_token_id=int(bos) if isinstance(bos, int) else None,
        stored_dtype=stored,
        raw=dict(raw),
    )


def _parse_llama(raw):
    return parse_dense_decoder(raw, architecture="LlamaForCausalLM", default_qkv_bias=False)


def _parse_qwen2(raw):
    return parse_dense_decoder(raw, architecture="Qwen2ForCausalLM", default_qkv_bias=True)


register_architecture("LlamaForCausalLM", _parse_llama, model_type="llama")
register_architecture("Qwen2ForCausalLM", _parse_qwen2, model_type="qwen2")
