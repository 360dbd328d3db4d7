"""The 8B-class shape (Llama-3.1-8B layer sizes: hidden 4096, 32 heads, 8 kv heads, head 128,
intermediate 14336, vocabulary 128256, rope theta 500000 with llama3 scaling), two layers,
random weights N(0, 0.02): logits of the engine against the plain implementation, in 32-bit
and in bfloat16, whole, in portions, token by token and mixed; and rotation at far positions."""
import pytest
import torch

import tiny
from plain_model import plain_logits

pytestmark = pytest.mark.gpu

RAW = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "intermediate_size": 14336, "num_hidden_layers": 2, "vocab_size": 128256,
    "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
}


@pytest.fixture(scope="module")
def weights():
    from blackwellllm_b200.weights.random_init import model_param_specs, random_tensors
    W = random_tensors(model_param_specs(RAW), seed=3, std=0.02, dtype=torch.bfloat16)
    return W  # bfloat16 values: both dtypes of the engine and the plain implementation use the same numbers


@pytest.fixture(scope="module")
def case(weights):
    ids_a = tiny.prompt(75, RAW["vocab_size"], 11)
    ids_b = tiny.prompt(40, RAW["vocab_size"], 12)
    with torch.no_grad():
        ref = {"a": plain_logits(RAW, weights, ids_a, dtype=torch.float64),
               "b": plain_logits(RAW, weights, ids_b, dtype=torch.float64)}
    return {"a": ids_a, "b": ids_b}, ref


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_8b_shape_every_way_of_cutting(weights, case, dtype):
    from blackwellllm_b200 import Engine, StepEntry
    ids, ref = case
    eng = Engine.from_tensors(RAW, weights, dtype=dtype, page_size=16, max_tokens=512, max_requests=4)
    tol = tiny.TOL[dtype]

    def check(rows, rid, start):
        r = ref[rid][start:start + rows.shape[0]]
        err = float((rows.double().cpu() - r).abs().max()) / float(ref[rid].abs().max())
        assert err <= tol, (rid, start, err)

    # whole
    a = ids["a"]
    check(eng.step([StepEntry("w", a, list(range(len(a))))]), "a", 0)
    eng.end_request("w")
    # portions of changing size, then token by token
    at = 0
    for n in (17, 2, 30, 3):
        check(eng.step([StepEntry("p", a[at:at + n], list(range(n)))]), "a", at)
        at += n
    while at < len(a):
        check(eng.step([StepEntry("p", [a[at]], [0])]), "a", at)
        at += 1
    # mixed: b's prompt in two portions beside a's decode tokens (request "p" rewound by 10 tokens)
    eng.cache.truncate("p", len(a) - 10)
    b = ids["b"]
    out = eng.step([StepEntry("p", [a[-10]], [0]), StepEntry("q", b[:25], list(range(25)))])
    check(out[:1], "a", len(a) - 10)
    check(out[1:], "b", 0)
    out = eng.step([StepEntry("q", b[25:], list(range(15))), StepEntry("p", [a[-9]], [0])])
    check(out[:15], "b", 25)
    check(out[15:], "a", len(a) - 9)


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    """The same weights (same seed, same tensor order) as a model folder, stored in bfloat16; the 32-bit
    replay converts them at load."""
    from blackwellllm_b200.weights.random_init import write_random_model
    return write_random_model(str(tmp_path_factory.mktemp("llama8b_shape")), RAW, seed=3, std=0.02, dtype="bfloat16")


@pytest.fixture(scope="module")
def replay_case(weights):
    """Six requests of 40 to 200 tokens and their plain logits (float64 through torch on the GPU: the
    vocabulary of 128,256 makes the CPU too slow for the suite's minutes)."""
    lengths = [40, 200, 97, 130, 65, 150]
    reqs = {f"r{i}": tiny.prompt(n, RAW["vocab_size"], 300 + i) for i, n in enumerate(lengths)}
    with torch.no_grad():
        plain = {rid: plain_logits(RAW, weights, ids, dtype=torch.float64, device="cuda:0") for rid, ids in reqs.items()}
    torch.cuda.empty_cache()
    return reqs, plain


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("family", ["mixed", "tail"])
def test_8b_shape_replay_mixed_with_page_reuse_and_tail(folder, replay_case, dtype, family):
    """bin/trace_run at the 8B shape: up to four live requests, portions of some beside decoded tokens of
    others, in a pool of 512 tokens for requests that need 960 (pages are used again); and each request
    with its last 32 tokens one by one."""
    import replay
    reqs, plain = replay_case
    if family == "mixed":
        max_tokens = 512
        steps = replay.trace_mixed(reqs, max_tokens, seed=5)
        assert max(len(s["entries"]) for s in steps) >= 3
    else:
        steps, max_tokens = replay.trace_tail(reqs)
    rows = replay.run_trace(folder, dtype, steps, max_tokens, RAW["vocab_size"], page_size=16, timeout=900)
    replay.compare(rows, plain, tiny.TOL[dtype], label=f"8B shape (2 layers) {dtype} {family}",
                   min_cosine=tiny.MIN_COSINE[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_8b_shape_long_prompt_in_portions_then_decode_from_the_graph(weights, dtype):
    """The benchmarked path at its lengths: a prompt of 4,200 tokens in portions of 2,048 + 2,048 + 104, then
    32 tokens decoded one by one from the CUDA graph; logits at the edges of the portions and at every
    decoded position against the plain implementation (computed once for the whole sequence, asked for
    those rows only)."""
    from blackwellllm_b200 import Engine, StepEntry
    from blackwellllm_b200.kernels import ops
    ids = tiny.prompt(4232, RAW["vocab_size"], 41)
    cuts = [(0, 2048), (2048, 4096), (4096, 4200)]
    wanted = {(0, 2048): [0, 1, 63, 64, 1000, 2047], (2048, 4096): [2048, 2049, 3000, 4095], (4096, 4200): [4096, 4199]}
    rows = [p for c in cuts for p in wanted[c]] + list(range(4200, 4232))
    with torch.no_grad():
        ref = plain_logits(RAW, weights, ids, dtype=torch.float64, rows=rows, device="cuda:0")
    torch.cuda.empty_cache()
    ref_of = {p: ref[i] for i, p in enumerate(rows)}
    scale = float(ref.abs().max())
    eng = Engine.from_tensors(RAW, weights, dtype=dtype, page_size=16, max_tokens=4352, max_requests=2,
                              max_batch_tokens=2048)
    worst = 0.0
    for a, b in cuts:
        out = eng.step([StepEntry("a", ids[a:b], [p - a for p in wanted[(a, b)]])]).double().cpu()
        for i, p in enumerate(wanted[(a, b)]):
            worst = max(worst, float((out[i] - ref_of[p]).abs().max()) / scale)
    for p in range(4200, 4232):
        out = eng.step([StepEntry("a", [ids[p]], [0])])[0].double().cpu()
        worst = max(worst, float((out - ref_of[p]).abs().max()) / scale)
    assert eng.graph_kernel_count(1) > 0
    assert worst <= tiny.TOL[dtype], worst
    assert ops.gemm_tc_status() == 0 and ops.attention_tc_status() == 0


def test_rope_scaling_at_far_positions():
    """llama3 scaling and theta 500000 at positions up to 16,640 (where float32 angles are coarse):
    rotated queries and keys of the engine's kernel against the plain rotation."""
    from blackwellllm_b200.config.specs import Llama3RopeScaling
    from blackwellllm_b200.kernels import ops
    from blackwellllm_b200.parts.rope import rotary_inv_freq
    from plain_model import plain_inv_freq, plain_rope
    dev = "cuda:0"
    hd, nh, nkv = 128, 4, 2
    positions = [0, 1, 8191, 8192, 12345, 16639]
    T = len(positions)
    inv = rotary_inv_freq(500000.0, hd, Llama3RopeScaling(8.0, 1.0, 4.0, 8192)).to(dev)
    g = torch.Generator().manual_seed(0)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, generator=g)
    pos = torch.tensor(positions, dtype=torch.int32, device=dev)
    pages = 16640 // 16 + 1
    kp = torch.zeros(pages, nkv, 16, hd, device=dev)
    vp = torch.zeros_like(kp)
    table = torch.arange(pages, dtype=torch.int32, device=dev).repeat(T, 1)
    req = torch.arange(T, dtype=torch.int32, device=dev)
    tab = ops.rope_table(pos, inv, hd)
    q = ops.rope_append(qkv.to(dev), pos, req, table, inv, hd, kp, vp, nh, nkv, hd, table=tab)
    x = qkv.double().view(T, nh + 2 * nkv, hd)
    ref_inv = plain_inv_freq(hd, 500000.0, (8.0, 1.0, 4.0, 8192))
    q_ref = plain_rope(x[:, :nh], torch.tensor(positions), ref_inv).reshape(T, nh * hd)
    k_ref = plain_rope(x[:, nh:nh + nkv], torch.tensor(positions), ref_inv)
    assert float((q.double().cpu() - q_ref).abs().max()) < 1e-5
    for t, p in enumerate(positions):
        got = kp[p // 16, :, p % 16].double().cpu()
        assert float((got - k_ref[t]).abs().max()) < 1e-5


MID = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 320, "num_attention_heads": 5,
       "num_key_value_heads": 1, "head_dim": 64, "intermediate_size": 736, "num_hidden_layers": 2, "vocab_size": 1000,
       "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False}


@pytest.mark.parametrize("dtype,pairs", [("float32", 1), ("bfloat16", 1), ("bfloat16", 2)])
def test_steps_of_more_than_512_tokens(dtype, pairs):
    """Steps wide enough for the products to run on CTA pairs (rotary and cache append, SwiGLU and
    the residual sum in their epilogues; q/k/v bias): a prompt of 700 tokens whole, then in portions of
    530 + 170 beside another request, against the plain implementation at every position."""
    from blackwellllm_b200 import Engine, StepEntry
    from blackwellllm_b200.kernels import ops
    from blackwellllm_b200.weights.random_init import model_param_specs, random_tensors
    before = ops.gemm_pair_mode(pairs)      # 2: every product that can runs on CTA pairs, whatever the estimate says
    try:
        _steps_of_more_than_512_tokens(dtype)
    finally:
        ops.gemm_pair_mode(before if before >= 0 else 1)


def _steps_of_more_than_512_tokens(dtype):
    from blackwellllm_b200 import Engine, StepEntry
    from blackwellllm_b200.weights.random_init import model_param_specs, random_tensors
    W = random_tensors(model_param_specs(MID), seed=21, std=0.05, bias_std=0.3,
                       dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    ids = tiny.prompt(700, MID["vocab_size"], 31)
    other = tiny.prompt(60, MID["vocab_size"], 32)
    with torch.no_grad():
        ref = plain_logits(MID, W, ids, dtype=torch.float64)
        ref_o = plain_logits(MID, W, other, dtype=torch.float64)
    eng = Engine.from_tensors(MID, W, dtype=dtype, page_size=16, max_tokens=1600, max_requests=3, max_batch_tokens=1024)
    tol, scale = tiny.TOL[dtype], float(ref.abs().max())
    out = eng.step([StepEntry("w", ids, list(range(700)))]).double().cpu()
    assert float((out - ref).abs().max()) / scale <= tol
    out = eng.step([StepEntry("p", ids[:530], list(range(530))), StepEntry("o", other[:30], list(range(30)))]).double().cpu()
    assert float((out[:530] - ref[:530]).abs().max()) / scale <= tol
    assert float((out[530:] - ref_o[:30]).abs().max()) / scale <= tol
    out = eng.step([StepEntry("o", other[30:], list(range(30))), StepEntry("p", ids[530:], list(range(170)))]).double().cpu()
    assert float((out[:30] - ref_o[30:]).abs().max()) / scale <= tol
    assert float((out[30:] - ref[530:]).abs().max()) / scale <= tol
    from blackwellllm_b200.kernels import ops
    assert ops.gemm_tc_status() == 0 and ops.attention_tc_status() == 0
