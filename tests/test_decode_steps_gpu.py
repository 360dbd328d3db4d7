"""Decode-only steps (one token per live request) at head sizes where the decode attention makes its own
queries, keys and values from the unsummed q/k/v product, and at sizes where it does not: random tiny
configurations (head sizes 32 to 256, partial rotary, llama3 bands, biases, pages of 8 to 64 and of 24), the
prompts whole and then the last tokens one per request and step, with and without CUDA graphs, every logit
row against the plain implementation."""
import random

import pytest
import torch

import tiny
from plain_model import plain_logits

pytestmark = pytest.mark.gpu


def random_case(case):
    rng = random.Random(case)
    hd = rng.choice([64, 128, 192, 256, 32])
    nkv = rng.choice([1, 2, 3, 4, 8])
    nh = nkv * rng.choice([1, 2, 4, 7, 8, 16])
    qwen = rng.random() < 0.5
    raw = {"architectures": ["Qwen2ForCausalLM" if qwen else "LlamaForCausalLM"], "model_type": "qwen2" if qwen else "llama",
           "hidden_size": rng.choice([64, 136, 264]), "num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd,
           "intermediate_size": rng.choice([80, 176, 400]), "num_hidden_layers": rng.choice([1, 2, 3]),
           "vocab_size": rng.choice([130, 500]), "rope_theta": rng.choice([1e4, 5e5]), "rms_norm_eps": 1e-5,
           "tie_word_embeddings": rng.random() < 0.3}
    if rng.random() < 0.4:
        raw["partial_rotary_factor"] = rng.choice([0.25, 0.5])
    if rng.random() < 0.3:
        raw["rope_scaling"] = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                               "original_max_position_embeddings": 32}
    page = rng.choice([8, 16, 32, 64, 24])
    graphs = rng.random() < 0.5
    tail = rng.choice([3, 20, 40])
    lens = [rng.choice([tail + 1, 64 + tail, 65 + tail, 130, 300, 700]) for _ in range(rng.randint(1, 4))]
    return raw, page, graphs, tail, lens


@pytest.mark.parametrize("case", range(24))
def test_decode_only_steps_against_the_plain_model(case):
    run_case(case)


@pytest.mark.parametrize("sums_open,own_rotation", [(False, False), (False, True), (True, False)])
@pytest.mark.parametrize("case", [1, 4, 9, 16])
def test_decode_only_steps_with_the_switches_off(case, sums_open, own_rotation, monkeypatch):
    """The paths behind the switches stay alive: every product sums its own K splits (BW_DEFER_SUMS=0) and / or
    the rotation kernel runs in decode-only steps too (BW_ATTN_FUSED_ROPE=0)."""
    from blackwellllm_b200.kernels import ops
    monkeypatch.setattr(ops, "DEFER_SUMS", sums_open)
    monkeypatch.setenv("BW_ATTN_FUSED_ROPE", "1" if own_rotation else "0")
    run_case(case)


def run_case(case):
    from blackwellllm_b200 import Engine, StepEntry
    from blackwellllm_b200.kernels import ops
    from blackwellllm_b200.weights.random_init import model_param_specs, random_tensors
    raw, page, graphs, tail, lens = random_case(case)
    W = random_tensors(model_param_specs(raw), seed=case, std=0.05, bias_std=0.2, dtype=torch.bfloat16)
    prompts = [tiny.prompt(n, raw["vocab_size"], case * 10 + i) for i, n in enumerate(lens)]
    refs = [plain_logits(raw, W, p, dtype=torch.float64) for p in prompts]
    eng = Engine.from_tensors(raw, W, dtype="bfloat16", page_size=page, max_tokens=sum(lens) + 128 * len(lens) + 256,
                              max_requests=4, max_batch_tokens=4096, cuda_graphs=graphs)
    err = 0.0

    def check(out, at):
        nonlocal err
        for i, ref in enumerate(refs):
            err = max(err, float((out[i] - ref[at(i)]).abs().max()) / float(ref.abs().max()))

    out = eng.step([StepEntry(i, p[:len(p) - tail], [len(p) - tail - 1]) for i, p in enumerate(prompts)]).double().cpu()
    check(out, lambda i: lens[i] - tail - 1)
    for k in range(tail):
        out = eng.step([StepEntry(i, [p[len(p) - tail + k]], [0]) for i, p in enumerate(prompts)]).double().cpu()
        check(out, lambda i: lens[i] - tail + k)
    assert err <= tiny.TOL["bfloat16"], (raw, page, graphs, lens, err)
    assert ops.pending_target() is None
    assert ops.gemm_tc_status() == 0
