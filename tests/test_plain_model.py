"""The plain implementation checked against itself and against hand-worked cases
(no GPU): it is the oracle of every other test, so its parts are pinned here."""
import math

import torch

import tiny
from plain_model import (plain_attention, plain_attention_tail, plain_config, plain_greedy, plain_inv_freq, plain_logits, plain_rmsnorm,
                         plain_rope, plain_swiglu)
from plain_sampling import plain_log_prob, plain_repetition_penalty, plain_sample


def test_config_defaults():
    c = plain_config({"hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "intermediate_size": 8,
                      "num_hidden_layers": 1, "vocab_size": 10, "model_type": "qwen2"})
    assert c["hd"] == 16 and c["eps"] == 1e-6 and c["theta"] == 10000.0 and c["bias"] is True and c["tie"] is False


def test_rmsnorm_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    y = plain_rmsnorm(x, torch.tensor([2.0, 0.5], dtype=torch.float64), 0.0)
    r = 1 / math.sqrt(12.5)
    assert torch.allclose(y, torch.tensor([[3 * r * 2, 4 * r * 0.5]], dtype=torch.float64))


def test_rope_is_identity_at_position_zero_and_a_rotation_elsewhere():
    inv = plain_inv_freq(8, 10000.0, None)
    x = torch.randn(3, 2, 8, dtype=torch.float64)
    y = plain_rope(x, torch.tensor([0, 5, 9]), inv)
    assert torch.equal(y[0], x[0])
    assert torch.allclose(y.pow(2).sum(-1), x.pow(2).sum(-1))       # rotations keep the norm
    # relative property: <rope(q, m), rope(k, n)> depends on m - n only
    q, k = torch.randn(1, 1, 8, dtype=torch.float64), torch.randn(1, 1, 8, dtype=torch.float64)
    a = (plain_rope(q, torch.tensor([7]), inv) * plain_rope(k, torch.tensor([3]), inv)).sum()
    b = (plain_rope(q, torch.tensor([14]), inv) * plain_rope(k, torch.tensor([10]), inv)).sum()
    assert abs(float(a - b)) < 1e-5


def test_llama3_bands():
    inv = plain_inv_freq(64, 500000.0, (8.0, 1.0, 4.0, 8192))
    base = plain_inv_freq(64, 500000.0, None)
    wl = 2 * math.pi / base
    assert torch.equal(inv[wl < 2048], base[wl < 2048])
    assert torch.allclose(inv[wl > 8192], base[wl > 8192] / 8)
    mid = (wl >= 2048) & (wl <= 8192)
    assert bool(mid.any()) and bool(((inv[mid] < base[mid]) & (inv[mid] > base[mid] / 8)).all())


def test_attention_causal_gqa_and_window():
    T, nh, nkv, hd = 5, 4, 2, 4
    q, k, v = (torch.randn(T, n, hd, dtype=torch.float64) for n in (nh, nkv, nkv))
    o = plain_attention(q, k, v)
    assert torch.allclose(o[0], v[0].repeat_interleave(2, dim=0))      # the first token sees itself only
    # by hand for the last token, head 3 (kv head 1)
    s = (k[:, 1] @ q[4, 3]) * hd ** -0.5
    assert torch.allclose(o[4, 3], torch.softmax(s, 0) @ v[:, 1])
    w1 = plain_attention(q, k, v, window=1)
    assert torch.allclose(w1, v.repeat_interleave(2, dim=1))           # window 1: each token sees itself
    w3 = plain_attention(q, k, v, window=3)
    s3 = (k[2:5, 0] @ q[4, 0]) * hd ** -0.5
    assert torch.allclose(w3[4, 0], torch.softmax(s3, 0) @ v[2:5, 0])


def test_attention_tail_is_the_tail_of_the_whole():
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(70, n, 8, generator=g, dtype=torch.float64) for n in (6, 2, 2))
    for window in (None, 9):
        whole = plain_attention(q, k, v, window=window)
        for n in (1, 13, 70):
            tail = plain_attention_tail(q[70 - n:], k, v, window=window, rows_at_once=5)
            assert float((tail - whole[70 - n:]).abs().max()) < 1e-12
    rows = plain_logits(tiny.TINY_QWEN, _tiny_weights(), list(range(9)), rows=[8, 2])
    full = plain_logits(tiny.TINY_QWEN, _tiny_weights(), list(range(9)))
    assert float((rows - full[[8, 2]]).abs().max()) < 1e-12


def _tiny_weights():
    from blackwellllm_b200.weights.random_init import model_param_specs, random_tensors
    return random_tensors(model_param_specs(tiny.TINY_QWEN), seed=1, std=0.05, bias_std=0.1, dtype=torch.float32)


def test_swiglu_by_hand():
    g, u = torch.tensor([0.0, 1.0, -2.0], dtype=torch.float64), torch.tensor([5.0, 2.0, 3.0], dtype=torch.float64)
    want = torch.tensor([0.0, 2 / (1 + math.exp(-1)), -6 / (1 + math.exp(2))], dtype=torch.float64)
    assert torch.allclose(plain_swiglu(g, u), want)


def test_logits_prefix_property_and_greedy():
    """Causality of the whole model: logits of a prefix equal the first rows of the
    logits of the longer sequence."""
    from blackwellllm_b200.weights.random_init import model_param_specs, random_tensors
    for name in ("llama", "qwen", "llama3", "partial"):
        raw, kw, _ = tiny.CONFIGS[name]
        W = random_tensors(model_param_specs(raw), kw["seed"], kw["std"], kw["bias_std"], dtype=torch.float32)
        ids = tiny.prompt(23, raw["vocab_size"], 1)
        full = plain_logits(raw, W, ids)
        assert full.shape == (23, raw["vocab_size"])
        assert torch.allclose(plain_logits(raw, W, ids[:9]), full[:9], atol=1e-12)
        nxt = plain_greedy(raw, W, ids, 2)
        assert nxt[0] == int(full[-1].argmax())
        if "partial_rotary_factor" in raw:   # the rotated span matters, and a factor of 1 is the default
            whole = {k: v for k, v in raw.items() if k != "partial_rotary_factor"}
            assert float((plain_logits(whole, W, ids) - full).abs().max()) > 1e-3 * float(full.abs().max())
            assert torch.equal(plain_logits(dict(whole, partial_rotary_factor=1.0), W, ids), plain_logits(whole, W, ids))


def test_plain_sampler():
    lg = torch.log(torch.tensor([0.1, 0.6, 0.3]))
    assert plain_sample(lg, 0.0, 1.0, 0.99)[0] == 1
    assert [plain_sample(lg, 1.0, 1.0, u)[0] for u in (0.05, 0.5, 0.95)] == [0, 1, 2]
    assert [plain_sample(lg, 1.0, 0.7, u)[0] for u in (0.05, 0.5, 0.95)] == [1, 1, 2]   # nucleus {1, 2}
    assert plain_sample(lg, 1.0, 0.5, 0.9)[0] == 1                                       # nucleus {1}


def test_plain_repetition_penalty_and_log_prob():
    # the reference's own test vectors (tests/validation/test_sampling.cpp:83-140): 4 -> 4 / 1.15, -4 -> -4 * 1.15,
    # an id that occurs many times is penalized once, ids outside the vocabulary and a penalty <= 1 do nothing
    lg = torch.zeros(32)
    lg[10], lg[20] = 4.0, -4.0
    out = plain_repetition_penalty(lg, [10, 20, 10, 10, -1, 99], 1.15)
    assert float(out[10]) == float(torch.tensor(4.0) / 1.15) and float(out[20]) == float(torch.tensor(-4.0) * 1.15)
    assert float(out.abs().sum()) == float(out[10].abs() + out[20].abs())
    assert torch.equal(plain_repetition_penalty(lg, [10, 20], 1.0), lg)
    probs = torch.tensor([0.1, 0.6, 0.3])
    assert abs(plain_log_prob(probs.log() + 3.0, 1) - float(torch.log(torch.tensor(0.6)))) < 1e-6
