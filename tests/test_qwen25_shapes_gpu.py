"""The layer sizes of Qwen2.5-7B (hidden 3584, 28 heads in 4 groups, intermediate 18944) and
Qwen2.5-14B (hidden 5120, 40 heads in 8 groups, intermediate 13824), vocabulary 152064, q/k/v bias,
one layer with random weights: logits of the engine against the plain implementation, in 32-bit and
in bfloat16, for a step of 700 tokens, portions down to two tokens, mixed steps and single tokens.
None of these widths is a power of two, and the products have other numbers of tiles than the
Llama-3.1-8B sizes."""
import pytest
import torch

import tiny
from plain_model import plain_logits

pytestmark = pytest.mark.gpu

SHAPES = {
    "qwen2.5-7b": dict(hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, head_dim=128,
                       intermediate_size=18944, vocab_size=152064),
    "qwen2.5-14b": dict(hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, head_dim=128,
                        intermediate_size=13824, vocab_size=152064),
}


@pytest.fixture(scope="module", params=list(SHAPES))
def case(request):
    from blackwellllm_b200.weights.random_init import model_param_specs, random_tensors
    raw = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=1, rope_theta=1e6,
               rms_norm_eps=1e-6, tie_word_embeddings=False, **SHAPES[request.param])
    W = random_tensors(model_param_specs(raw), seed=4, std=0.02, bias_std=0.1, dtype=torch.bfloat16)
    ids = {"a": tiny.prompt(700, raw["vocab_size"], 1), "b": tiny.prompt(90, raw["vocab_size"], 2)}
    with torch.no_grad():
        ref = {k: plain_logits(raw, W, v, dtype=torch.float64) for k, v in ids.items()}
    return raw, W, ids, ref


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_qwen25_shapes_every_way_of_cutting(case, dtype):
    from blackwellllm_b200 import Engine, StepEntry
    from blackwellllm_b200.kernels import ops
    raw, W, ids, ref = case
    eng = Engine.from_tensors(raw, W, dtype=dtype, page_size=16, max_tokens=2048, max_requests=4,
                              max_batch_tokens=1024)
    tol = tiny.TOL[dtype]

    def check(rows, rid, start):
        r = ref[rid][start:start + rows.shape[0]]
        err = float((rows.double().cpu() - r).abs().max()) / float(ref[rid].abs().max())
        assert err <= tol, (rid, start, rows.shape[0], err)

    a, b = ids["a"], ids["b"]
    check(eng.step([StepEntry("w", a, list(range(len(a))))]), "a", 0)          # one step of 700 tokens
    eng.end_request("w")
    at = 0
    for n in (300, 257, 100, 17, 2):
        check(eng.step([StepEntry("p", a[at:at + n], list(range(n)))]), "a", at)
        at += n
    # mixed: b's prompt in two portions beside a's next tokens
    out = eng.step([StepEntry("p", [a[at]], [0]), StepEntry("q", b[:64], list(range(64)))])
    check(out[:1], "a", at)
    check(out[1:], "b", 0)
    at += 1
    out = eng.step([StepEntry("q", b[64:], list(range(26))), StepEntry("p", a[at:at + 2], [0, 1])])
    check(out[:26], "b", 64)
    check(out[26:], "a", at)
    at += 2
    while at < len(a):                                                         # token by token to the end
        check(eng.step([StepEntry("p", [a[at]], [0])]), "a", at)
        at += 1
    assert ops.gemm_tc_status() == 0 and ops.attention_tc_status() == 0
