"""Tiny configurations of the architecture for the tests.  They differ in every
size and option: heads and groups, sizes that are no power of two, layers,
vocabulary, the norms' eps, rope base and scaling, the rotated span of a head,
bias, tied head."""
import os

import torch

from blackwellllm_b200.weights.random_init import write_random_model

TINY_LLAMA = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "intermediate_size": 176, "num_hidden_layers": 2, "vocab_size": 256,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "max_position_embeddings": 2048,
}
TINY_QWEN = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32,
    "intermediate_size": 256, "num_hidden_layers": 3, "vocab_size": 384,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 4096,
}
# rope scaling with all three wavelength bands inside a head of 32 channels
TINY_LLAMA3 = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 80, "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 32,
    "intermediate_size": 136, "num_hidden_layers": 1, "vocab_size": 300,
    "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 32},
    "max_position_embeddings": 1024,
}
# half of each head rotated (partial_rotary_factor, src/core/config.cpp:194-201); six heads in three groups
TINY_PARTIAL = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 72, "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 48,
    "intermediate_size": 200, "num_hidden_layers": 2, "vocab_size": 500,
    "rope_theta": 20000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "partial_rotary_factor": 0.5, "max_position_embeddings": 2048,
}

CONFIGS = {
    "llama": (TINY_LLAMA, dict(seed=0, std=0.02, bias_std=None), 16),
    "qwen": (TINY_QWEN, dict(seed=1, std=0.05, bias_std=0.1), 8),
    "llama3": (TINY_LLAMA3, dict(seed=7, std=0.04, bias_std=None), 16),
    "partial": (TINY_PARTIAL, dict(seed=11, std=0.05, bias_std=None), 32),
}


def make_folder(name: str, dtype: str, root: str) -> str:
    raw, kw, _ = CONFIGS[name]
    d = os.path.join(root, f"{name}-{dtype}")
    if not os.path.isdir(d):
        write_random_model(d, raw, dtype=dtype, **kw)
    return d


def prompt(n: int, vocab: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def scale_of(ref: torch.Tensor) -> float:
    return float(ref.abs().max())


# tolerances, relative to the largest logit magnitude of the compared rows
# (bfloat16: the worst measured over all configurations and ways of cutting is 7e-3; a single wrong page
# in one layer of a tiny model moves the logits by more than this bound: tests/test_engine_gpu.py)
TOL = {"float32": 1e-4, "bfloat16": 1.5e-2}
MIN_COSINE = {"float32": 0.999999, "bfloat16": 0.999}
