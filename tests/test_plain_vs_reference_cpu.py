"""The plain implementation against the reference project's own CPU kernels.

``tests/golden/reference_cpu.json`` holds inputs and outputs of
fxslava/BlackwellLLM's ``tests/common/cpu_reference.h`` (rope + cache append,
single-query attention, RMSNorm, SwiGLU, embedding, argmax), made by
``tests/golden/make_golden.cpp`` (see ``make_golden.sh``).  The reference's whole
model cannot run here (it needs a GPU and its author's checkpoints), so the
comparison is part by part, and then once for a whole tiny decoder that
``tests/golden/make_layer_golden.cpp`` composes only of those CPU kernels in the
order of the reference's layer loop (``reference_layer.json``): that pins the
composition (bias before the rotation, the residual sums, which query heads read
which kv head, the tied head).  ``reference_rope_scaling.json`` holds the
reference's own llama3 frequency rescaling (``apply_rope_scaling`` of its
``src/kernels/rope.cuh``, compiled for the host by ``make_rope_scaling_golden.cpp``).

Rope, attention, embedding and argmax are float32 code in the reference without
bfloat16 latches: they must agree to float32 rounding.  Its RMSNorm and SwiGLU snap
values to the bfloat16 grid (rmsnorm.cu:133-138, swiglu.cu:23-34): the exact
arithmetic agrees with them to two bfloat16 roundings.
"""
import json
import os

import torch

from plain_model import (plain_attention, plain_embedding, plain_inv_freq, plain_logits, plain_rmsnorm, plain_rope,
                         plain_swiglu)

HERE = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(HERE, "golden", "reference_cpu.json")) as f:
    G = json.load(f)


def t(name, *shape):
    return torch.tensor(G[name], dtype=torch.float64).reshape(*shape)


def test_rope_matches_reference_cpu():
    nh, nkv, hd, T = G["nh"], G["nkv"], G["hd"], G["T"]
    inv = plain_inv_freq(hd, G["theta"], None)
    pos = torch.arange(T)
    q = plain_rope(t("q_in", T, nh, hd), pos, inv)
    k = plain_rope(t("k_in", T, nkv, hd), pos, inv)
    assert float((q - t("q_rot", T, nh, hd)).abs().max()) < 2e-6
    assert float((k - t("k_rot", T, nkv, hd)).abs().max()) < 2e-6


def test_attention_matches_reference_cpu_at_every_position():
    nh, nkv, hd, T = G["nh"], G["nkv"], G["hd"], G["T"]
    # the reference attends position by position over its cache; the plain function does
    # the whole causal sequence at once: row p must equal the reference's output at p
    o = plain_attention(t("q_rot", T, nh, hd), t("k_rot", T, nkv, hd), t("v_in", T, nkv, hd))
    assert float((o - t("attn", T, nh, hd)).abs().max()) < 2e-6


def test_rmsnorm_and_swiglu_match_reference_cpu_up_to_its_bf16_latches():
    y = plain_rmsnorm(t("norm_x", 3, 24), t("norm_w", 24), 1e-5)
    ref = t("norm_y", 3, 24)
    assert float(((y - ref).abs() / ref.abs().clamp_min(1e-3)).max()) < 2 * 2 ** -8
    s = plain_swiglu(t("swiglu_g", 40), t("swiglu_u", 40))
    ref = t("swiglu_y", 40)
    assert float((s - ref).abs().max()) < 3 * 2 ** -8 * float(ref.abs().max())


def test_embedding_and_argmax_match_reference_cpu():
    out = plain_embedding(t("embed_table", 5, 4), [4, 0, 2])
    assert torch.equal(out, t("embed_out", 3, 4))
    lg = t("argmax_logits", 5)
    best = int((lg == lg.max()).nonzero()[0])        # the lowest index among the maxima
    assert best == G["argmax"] == 1


def _golden(name):
    with open(os.path.join(HERE, "golden", name)) as f:
        return json.load(f)


def test_llama3_frequency_bands_match_the_references_own_function():
    """All three wavelength bands, head sizes 32 and 128, two rope bases: the plain implementation's
    frequencies and the product's table against ``apply_rope_scaling`` of the reference (float32 there)."""
    from blackwellllm_b200.config.specs import Llama3RopeScaling
    from blackwellllm_b200.parts.rope import rotary_inv_freq
    seen = set()
    for c in _golden("reference_rope_scaling.json")["cases"]:
        scaled = torch.tensor(c["scaled"], dtype=torch.float64)
        plain = plain_inv_freq(c["head_dim"], c["theta"], (c["factor"], c["low"], c["high"], c["orig"]))
        ours = rotary_inv_freq(c["theta"], c["head_dim"], Llama3RopeScaling(c["factor"], c["low"], c["high"], int(c["orig"])))
        assert float(((plain - scaled).abs() / scaled).max()) < 2e-6
        assert float(((ours.double() - scaled).abs() / scaled).max()) < 2e-6
        unscaled = plain_inv_freq(c["head_dim"], c["theta"], None)
        assert float(((unscaled - torch.tensor(c["plain"], dtype=torch.float64)).abs() / unscaled).max()) < 2e-6
        seen |= set(c["band"])
    assert seen == {0, 1, 2}


def test_whole_tiny_decoder_matches_the_composition_of_reference_cpu_kernels():
    """Embedding, a layer with q/k/v bias and two query heads per kv head, final norm and tied head at six
    positions: the plain implementation on the same weights against the logits that the reference's CPU
    kernels give when composed in its engine's order.  The reference's norm and SwiGLU snap values to the
    bfloat16 grid (four latches a position on the way to the logits); the plain arithmetic is exact."""
    L = _golden("reference_layer.json")
    H, nh, nkv, hd, I, V, T = (L[k] for k in ("H", "nh", "nkv", "hd", "I", "V", "T"))
    raw = {"model_type": "qwen2", "hidden_size": H, "num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd,
           "intermediate_size": I, "num_hidden_layers": 1, "vocab_size": V, "rope_theta": L["theta"],
           "rms_norm_eps": L["eps"], "tie_word_embeddings": True}

    def w(name, *shape):
        return torch.tensor(L[name], dtype=torch.float64).reshape(*shape)

    p = "model.layers.0."
    W = {"model.embed_tokens.weight": w("embed", V, H), "model.norm.weight": w("norm_f", H),
         p + "input_layernorm.weight": w("norm1", H), p + "post_attention_layernorm.weight": w("norm2", H),
         p + "self_attn.q_proj.weight": w("wq", nh * hd, H), p + "self_attn.k_proj.weight": w("wk", nkv * hd, H),
         p + "self_attn.v_proj.weight": w("wv", nkv * hd, H), p + "self_attn.q_proj.bias": w("bq", nh * hd),
         p + "self_attn.k_proj.bias": w("bk", nkv * hd), p + "self_attn.v_proj.bias": w("bv", nkv * hd),
         p + "self_attn.o_proj.weight": w("wo", H, nh * hd), p + "mlp.gate_proj.weight": w("wg", I, H),
         p + "mlp.up_proj.weight": w("wu", I, H), p + "mlp.down_proj.weight": w("wd", H, I)}
    ref = w("logits", T, V)
    got = plain_logits(raw, W, L["tokens"])
    scale = float(ref.abs().max())
    err = float((got - ref).abs().max()) / scale
    assert err < 2 * 2 ** -8, err            # measured: 3.2e-3
    # the bound is that of the latches, not slack for a wrong composition: each of these changes breaks it
    no_bias = dict(W); no_bias[p + "self_attn.k_proj.bias"] = torch.zeros(nkv * hd, dtype=torch.float64)
    swapped = dict(W); swapped[p + "mlp.gate_proj.weight"], swapped[p + "mlp.up_proj.weight"] = W[p + "mlp.up_proj.weight"], W[p + "mlp.gate_proj.weight"]
    untied = dict(raw, tie_word_embeddings=False); W2 = dict(W); W2["lm_head.weight"] = W["model.embed_tokens.weight"].flip(0)
    for other in (plain_logits(raw, no_bias, L["tokens"]), plain_logits(raw, swapped, L["tokens"]),
                  plain_logits(untied, W2, L["tokens"]), plain_logits(dict(raw, num_key_value_heads=nkv, rope_theta=500.0), W, L["tokens"])):
        assert float((other - ref).abs().max()) / scale > 4 * 2 ** -8   # the smallest of them: 7e-2
