"""The configuration parser against the reference project's own loader.

``tests/golden/reference_config.json`` holds what fxslava/BlackwellLLM's ``ConfigLoader::load_from_json``
(src/core/config.cpp, compiled on the CPU by ``tests/golden/make_config_golden.sh``) read from the
tiny config.json files of ``tests/golden/config_cases.json``: sizes, defaults (eps 1e-6, theta 1e4,
q/k/v bias by model type, head size = hidden / heads), llama3 scaling keys and their defaults, and
the keys it demands.  This parser must read the same from the same files.  One deliberate
difference: an unknown rope scaling type is refused here, where the reference warns and runs the
unscaled rotation.
"""
import json
import os

import numpy as np
import pytest

from blackwellllm_b200.config.registry import parse_config

HERE = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(HERE, "golden", "reference_config.json")) as f:
    CASES = json.load(f)


def f32(x):
    return float(np.float32(x))


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_parser_reads_what_the_reference_reads(case):
    raw = case["config"]
    if "error" in case:
        assert "num_key_value_heads" in case["error"]           # the one refusal among the cases
        with pytest.raises(Exception, match="num_key_value_heads"):
            parse_config(raw)
        return
    ref = case["parsed"]
    if case["name"] == "unknown_rope_scaling":
        assert ref["rope_scaling_type"] == 0                     # the reference falls back to no scaling
        with pytest.raises(Exception, match="not supported"):
            parse_config(raw)
        return
    cfg = parse_config(raw)
    assert len(cfg.layers) == ref["num_layers"] and cfg.hidden_size == ref["hidden_dim"]
    assert cfg.vocab_size == ref["vocab_size"] and cfg.tie_word_embeddings == ref["tie_word_embeddings"]
    assert cfg.max_position_embeddings == ref["max_position_embeddings"]
    for layer in cfg.layers:
        att, ffn = layer.mixer, layer.ffn
        assert (att.num_heads, att.num_kv_heads, att.head_dim) == (ref["num_attention_heads"], ref["num_key_value_heads"],
                                                                   ref["head_dim"])
        assert att.qkv_bias == ref["has_qkv_bias"] and ffn.intermediate_size == ref["intermediate_dim"]
        assert f32(layer.mixer_norm.eps) == f32(ref["rms_norm_eps"]) and f32(layer.ffn_norm.eps) == f32(ref["rms_norm_eps"])
        rope = att.position
        assert rope.rotary_dim == ref["rotary_dim"] and f32(rope.theta) == f32(ref["rope_theta"])
        if ref["rope_scaling_type"] == 0:
            assert rope.scaling is None
        else:
            sc = rope.scaling
            assert (f32(sc.factor), f32(sc.low_freq_factor), f32(sc.high_freq_factor)) == \
                (f32(ref["rope_scaling_factor"]), f32(ref["rope_low_freq_factor"]), f32(ref["rope_high_freq_factor"]))
            assert float(sc.original_max_position_embeddings) == ref["rope_orig_max_pos"]
    assert f32(cfg.final_norm.eps) == f32(ref["rms_norm_eps"])
