"""Configuration parsing, the registry, safetensors IO and weight-binding errors (no GPU)."""
import json
import os
import struct

import pytest
import torch

import tiny
from blackwellllm_b200.config import ConfigError, load_config, parse_config, registered_architectures
from blackwellllm_b200.parts.base import ParamSpec
from blackwellllm_b200.weights.loader import WeightError, bind_tensors, check_names, kept_dtype, load_weights
from blackwellllm_b200.weights.random_init import model_param_specs, random_tensors, write_random_model
from blackwellllm_b200.weights.safetensors_io import SafetensorsError, index_folder, read_header, write_file


def test_registry_names():
    assert set(registered_architectures()) >= {"LlamaForCausalLM", "Qwen2ForCausalLM"}


def test_llama_defaults_follow_the_reference():
    raw = {"architectures": ["LlamaForCausalLM"], "hidden_size": 64, "num_attention_heads": 4,
           "num_key_value_heads": 2, "intermediate_size": 176, "num_hidden_layers": 2, "vocab_size": 256}
    c = parse_config(raw)
    a = c.layers[0].mixer
    assert (a.num_heads, a.num_kv_heads, a.head_dim) == (4, 2, 16)
    assert a.qkv_bias is False and a.window is None
    assert a.position.theta == 10000.0 and a.position.rotary_dim == 16 and a.position.scaling is None
    assert c.layers[0].mixer_norm.eps == 1e-6 and c.final_norm.eps == 1e-6
    assert c.tie_word_embeddings is False
    assert [e.layer for e in c.schedule] == [0, 1] and all(e.cache_of is None for e in c.schedule)


def test_qwen2_bias_default_and_tied():
    c = parse_config(tiny.TINY_QWEN)
    assert c.layers[0].mixer.qkv_bias is True and c.tie_word_embeddings is True
    assert c.layers[0].mixer.position.theta == 1e6
    c2 = parse_config(dict(tiny.TINY_QWEN, attention_bias=False))
    assert c2.layers[0].mixer.qkv_bias is False


def test_model_type_fallback():
    raw = dict(tiny.TINY_LLAMA)
    del raw["architectures"]
    assert parse_config(raw).architecture == "LlamaForCausalLM"


def test_llama3_scaling_keys():
    c = parse_config(tiny.TINY_LLAMA3)
    s = c.layers[0].mixer.position.scaling
    assert (s.factor, s.low_freq_factor, s.high_freq_factor, s.original_max_position_embeddings) == (8.0, 1.0, 4.0, 32)
    d = parse_config(dict(tiny.TINY_LLAMA, rope_scaling={"type": "llama3"}))
    s = d.layers[0].mixer.position.scaling
    assert (s.factor, s.low_freq_factor, s.high_freq_factor, s.original_max_position_embeddings) == (8.0, 1.0, 4.0, 8192)


@pytest.mark.parametrize("patch,msg", [
    ({"architectures": ["MambaForCausalLM"]}, "unsupported architecture"),
    ({"num_key_value_heads": 3}, "not a multiple"),
    ({"hidden_size": 0}, "positive integer"),
    ({"use_sliding_window": True}, "sliding"),
    ({"quantization_config": {"bits": 4}}, "quantiz"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, "not supported"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rms_norm_eps": 0}, "rms_norm_eps"),
])
def test_config_errors(patch, msg):
    with pytest.raises(ConfigError, match=msg):
        parse_config(dict(tiny.TINY_LLAMA, **patch))


def test_missing_required_keys_are_all_named():
    raw = dict(tiny.TINY_LLAMA)
    del raw["vocab_size"], raw["intermediate_size"]
    with pytest.raises(ConfigError) as e:
        parse_config(raw)
    assert "vocab_size" in str(e.value) and "intermediate_size" in str(e.value)


def test_load_config_errors(tmp_path):
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_config(str(tmp_path))


def test_random_model_folder_roundtrip(tmp_path):
    d = write_random_model(str(tmp_path / "m"), tiny.TINY_QWEN, seed=1, std=0.05, bias_std=0.1, dtype="bfloat16")
    cfg = load_config(d)
    ents = index_folder(d)
    specs = model_param_specs(cfg.raw)
    assert "lm_head.weight" not in ents  # tied: not written
    assert set(ents) == {n for n, s in specs.items() if not s.optional}
    assert all(e.dtype == torch.bfloat16 for e in ents.values())
    from safetensors.torch import load_file
    theirs = load_file(os.path.join(d, "model.safetensors"))
    ours = load_weights(d, specs, torch.bfloat16, torch.device("cpu"))
    for n in theirs:
        assert torch.equal(theirs[n], ours[n]), n
    g = theirs["model.layers.0.input_layernorm.weight"]
    assert torch.all(g == 1)
    b = theirs["model.layers.1.self_attn.k_proj.bias"].float()
    assert 0.03 < float(b.std()) < 0.3
    again = random_tensors(specs, 1, 0.05, 0.1, torch.bfloat16)
    assert torch.equal(again["model.embed_tokens.weight"], theirs["model.embed_tokens.weight"])
    other = random_tensors(specs, 2, 0.05, 0.1, torch.bfloat16)
    assert not torch.equal(other["model.embed_tokens.weight"], theirs["model.embed_tokens.weight"])


def test_weight_error_lists_everything(tmp_path):
    d = write_random_model(str(tmp_path / "m"), tiny.TINY_LLAMA, seed=0, dtype="float32")
    from safetensors.torch import load_file, save_file
    t = load_file(os.path.join(d, "model.safetensors"))
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.mlp.extra.weight"] = torch.zeros(3)
    t["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 60)
    save_file(t, os.path.join(d, "model.safetensors"))
    specs = model_param_specs(tiny.TINY_LLAMA)
    with pytest.raises(WeightError) as e:
        load_weights(d, specs, torch.float32, torch.device("cpu"))
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.mlp.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (64, 60), (64, 64))]
    s = str(err)
    for frag in ("missing (2)", "unexpected (1)", "wrong shape (1)", "expected [64, 64]"):
        assert frag in s


def test_unexpected_tensors_derived_buffers_and_the_switch(capsys):
    """A derived buffer that old exporters store is passed over with a note; any other tensor the model
    does not ask for is an error unless the caller says to ignore it."""
    specs = model_param_specs(tiny.TINY_LLAMA)
    t = random_tensors(specs, 0, dtype=torch.float32)
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    out = bind_tensors(t, specs, torch.float32, torch.device("cpu"))
    assert "model.layers.0.self_attn.rotary_emb.inv_freq" not in out and "passed over" in capsys.readouterr().err
    t["model.extra.weight"] = torch.zeros(3)
    with pytest.raises(WeightError) as e:
        bind_tensors(t, specs, torch.float32, torch.device("cpu"))
    assert e.value.unexpected == ["model.extra.weight"]
    out = bind_tensors(t, specs, torch.float32, torch.device("cpu"), ignore_unexpected=True)
    assert set(out) == {n for n, s_ in specs.items() if not s_.optional}
    assert "2 tensor(s)" in capsys.readouterr().err


def test_generation_config_adds_end_of_sequence_ids(tmp_path):
    d = str(tmp_path / "m")
    os.makedirs(d)
    raw = dict(tiny.TINY_LLAMA, eos_token_id=7)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(raw, f)
    assert load_config(d).eos_token_ids == (7,)
    with open(os.path.join(d, "generation_config.json"), "w") as f:
        json.dump({"eos_token_id": [9, 7, 11], "temperature": 0.6}, f)
    assert load_config(d).eos_token_ids == (9, 7, 11)
    with open(os.path.join(d, "generation_config.json"), "w") as f:
        json.dump({"eos_token_id": 3}, f)
    assert load_config(d).eos_token_ids == (3, 7)
    with open(os.path.join(d, "generation_config.json"), "w") as f:
        json.dump({"eos_token_id": "no"}, f)
    with pytest.raises(ConfigError, match="eos_token_id"):
        load_config(d)
    assert parse_config(dict(tiny.TINY_LLAMA, layernorm_epsilon=3e-7, rms_norm_eps=None) | {"rms_norm_eps": 2e-6}).layers[0].mixer_norm.eps == 2e-6
    alias = {k: v for k, v in tiny.TINY_LLAMA.items() if k != "rms_norm_eps"}
    assert parse_config(dict(alias, layernorm_epsilon=3e-7)).final_norm.eps == 3e-7


def test_tied_head_tolerates_a_stored_lm_head():
    specs = model_param_specs(tiny.TINY_QWEN)
    t = random_tensors(specs, 0, dtype=torch.float32)
    t["lm_head.weight"] = torch.zeros(384, 96)
    check_names("x", specs, t)  # no error
    untied = model_param_specs(tiny.TINY_LLAMA)
    t2 = random_tensors(untied, 0, dtype=torch.float32)
    del t2["lm_head.weight"]
    with pytest.raises(WeightError, match="lm_head.weight"):
        check_names("x", untied, t2)


def test_kept_dtypes():
    m, g, i = ParamSpec("w", (2, 2)), ParamSpec("g", (2,), role="gain"), ParamSpec("t", (2,), role="int_table")
    assert kept_dtype(m, torch.float32, torch.bfloat16) == torch.bfloat16
    assert kept_dtype(g, torch.float32, torch.bfloat16) == torch.float32   # stored in 32-bit: stays
    assert kept_dtype(g, torch.bfloat16, torch.bfloat16) == torch.bfloat16
    assert kept_dtype(g, torch.bfloat16, torch.float32) == torch.float32   # the 32-bit path
    assert kept_dtype(i, torch.int64, torch.bfloat16) == torch.int32
    with pytest.raises(WeightError, match="wrong type"):
        bind_tensors({"w": torch.zeros(2, 2, dtype=torch.int32)}, {"w": m}, torch.float32, torch.device("cpu"))


def test_safetensors_errors(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(SafetensorsError, match="shorter"):
        read_header(str(p))
    p.write_bytes(struct.pack("<Q", 10_000) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        read_header(str(p))
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)
    with pytest.raises(SafetensorsError, match="bad data_offsets"):
        read_header(str(p))
    with pytest.raises(SafetensorsError, match="neither"):
        index_folder(str(tmp_path / "nothing"))


def test_sharded_folder(tmp_path):
    a = {"x": torch.arange(6, dtype=torch.float32).reshape(2, 3)}
    b = {"y": torch.ones(4, dtype=torch.bfloat16)}
    write_file(str(tmp_path / "s1.safetensors"), a)
    write_file(str(tmp_path / "s2.safetensors"), b)
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"x": "s1.safetensors", "y": "s2.safetensors"}}))
    ents = index_folder(str(tmp_path))
    assert ents["x"].shape == (2, 3) and ents["y"].dtype == torch.bfloat16
    write_file(str(tmp_path / "s2.safetensors"), {"y": b["y"], "x": a["x"]})
    with pytest.raises(SafetensorsError, match="more than one shard"):
        index_folder(str(tmp_path))


def test_every_stored_type_and_odd_shapes_survive_the_file(tmp_path):
    """Writer and reader on every type the container names here, a tensor without dimensions, an empty
    one, and a file cut short after its header was written."""
    from blackwellllm_b200.weights.safetensors_io import TensorFiles
    ts = {"f32": torch.randn(3, 5), "bf16": torch.randn(7).to(torch.bfloat16), "f16": torch.randn(2, 2).half(),
          "f64": torch.randn(4, dtype=torch.float64), "i64": torch.arange(5), "i32": torch.arange(6, dtype=torch.int32).reshape(2, 3),
          "i16": torch.arange(3, dtype=torch.int16), "i8": torch.arange(-2, 2, dtype=torch.int8),
          "u8": torch.arange(3, dtype=torch.uint8), "bool": torch.tensor([True, False, True]),
          "scalar": torch.tensor(3.5), "empty": torch.empty(0, 4)}
    path = str(tmp_path / "all.safetensors")
    write_file(path, ts)
    entries = read_header(path)
    with TensorFiles() as files:
        got = {n: files.read(e) for n, e in entries.items()}
    assert set(got) == set(ts)
    for n, t in ts.items():
        assert got[n].dtype == t.dtype and got[n].shape == t.shape and torch.equal(got[n], t), n
    got["f32"].zero_()                                   # a copy of its own: writable, the file is closed
    with TensorFiles() as files:
        assert torch.equal(files.read(entries["f32"]), ts["f32"])
    # the file loses its tail after the header was read
    size = os.path.getsize(path)
    with open(path, "r+b") as f:
        f.truncate(size - 8)
    last = max(entries.values(), key=lambda e: e.begin + e.nbytes)
    with TensorFiles() as files, pytest.raises(SafetensorsError, match="short read"):
        files.read(last)
    with pytest.raises(SafetensorsError, match="data_offsets"):
        read_header(path)
