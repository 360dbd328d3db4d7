"""The plain implementation against the reference project's own CPU kernels.

``tests/golden/reference_cpu.json`` holds inputs and outputs of
fxslava/BlackwellLLM's ``tests/common/cpu_reference.h`` (rope + cache append,
single-query attention, RMSNorm, SwiGLU, embedding, argmax), made by
``tests/golden/make_golden.cpp`` (see ``make_golden.sh``).  The reference's whole
model cannot run here (it needs a GPU and its author's checkpoints), so the
comparison is part by part; the whole-model oracle rests on the formulas.

Rope, attention, embedding and argmax are float32 code in the reference without
bfloat16 latches: they must agree to float32 rounding.  Its RMSNorm and SwiGLU snap
values to the bfloat16 grid (rmsnorm.cu:133-138, swiglu.cu:23-34): the exact
arithmetic agrees with them to two bfloat16 roundings.
"""
import json
import os

import torch

from plain_model import (plain_attention, plain_embedding, plain_inv_freq, plain_rmsnorm, plain_rope, plain_swiglu)

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
