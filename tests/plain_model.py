"""Plain, slow implementation of the Llama/Qwen2 dense decoder: the tests' oracle.

Whole sequences, no cache, one function per part, torch tensor ops on the CPU in
float64 (or any dtype asked for).  It shares no code with the product package: it
reads config.json keys itself and takes weights as a dict of tensors by their
checkpoint names.

This file rests on the reference's formulas (cited per function as
file:line within fxslava/BlackwellLLM).  The reference's whole model needs a GPU
and cannot run here; its CPU kernels (tests/common/cpu_reference.h) and its
llama3 frequency rescaling (src/kernels/rope.cuh) can, and ``tests/golden/``
holds their outputs: part by part, and composed into one whole tiny decoder in
the order of the reference's layer loop, for the comparisons in
``test_plain_vs_reference_cpu.py``.  Where the reference rounds intermediate
values to the bfloat16 grid to mimic a bfloat16 PyTorch run (rmsnorm.cu:133-138,
swiglu.cu:23-34), this implementation does not: it is the exact arithmetic.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


# --------------------------------------------------------------------------- config

def plain_config(raw: dict) -> dict:
    """The sizes and constants of a model, with the reference's defaults.

    src/core/config.cpp:126-131 (required sizes), 144-145 (head_dim default),
    157 (rms_norm_eps default 1e-6), 158 (tie default false), 188 (rope_theta
    default 10000), 226-227 (qkv bias default: model_type == "qwen2"),
    263-273 (llama3 rope scaling keys and their defaults), 194-201 (the rotated
    span: head_dim x partial_rotary_factor, default 1, rounded down to even;
    the whole head if that leaves 0 or more than the head).
    """
    c = {
        "H": raw["hidden_size"], "nh": raw["num_attention_heads"],
        "nkv": raw["num_key_value_heads"], "I": raw["intermediate_size"],
        "L": raw["num_hidden_layers"], "V": raw["vocab_size"],
    }
    c["hd"] = raw.get("head_dim") or c["H"] // c["nh"]
    c["eps"] = raw.get("rms_norm_eps", 1e-6)
    c["theta"] = raw.get("rope_theta", 10000.0)
    c["bias"] = raw.get("attention_bias", raw.get("model_type") == "qwen2")
    c["tie"] = raw.get("tie_word_embeddings", False)
    rd = int(float(c["hd"]) * float(raw.get("partial_rotary_factor", 1.0)))
    c["rd"] = (rd if 0 < rd <= c["hd"] else c["hd"]) & ~1
    rs = raw.get("rope_scaling")
    c["scaling"] = None
    if rs is not None and rs.get("rope_type", rs.get("type")) == "llama3":
        c["scaling"] = (rs.get("factor", 8.0), rs.get("low_freq_factor", 1.0),
                        rs.get("high_freq_factor", 4.0),
                        rs.get("original_max_position_embeddings", 8192))
    return c


# --------------------------------------------------------------------------- parts

def plain_embedding(table: torch.Tensor, ids: Sequence[int]) -> torch.Tensor:
    """x[t, :] = E[id_t, :], no scaling (src/kernels/embedding.cu:45-69)."""
    return table[torch.as_tensor(list(ids), dtype=torch.long, device=table.device)]


def plain_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x / sqrt(mean(x^2) + eps) * w (src/kernels/rmsnorm.cu:107-120, 133-138,
    without the bfloat16 latches)."""
    r = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return x * r * w


def plain_inv_freq(head_dim: int, theta: float, scaling, rotary_dim: Optional[int] = None) -> torch.Tensor:
    """inv_j = theta ** (-2j / rotary_dim), then the llama3 wavelength bands
    (src/kernels/rope.cu:21-22; src/kernels/rope.cuh:24-38).  float64."""
    rd = rotary_dim or head_dim
    j = torch.arange(rd // 2, dtype=torch.float64)
    inv = 1.0 / (torch.tensor(float(theta), dtype=torch.float64) ** (2.0 * j / rd))
    if scaling is not None:
        factor, low, high, orig = scaling
        wavelen = 2.0 * math.pi / inv
        low_wavelen = orig / low
        high_wavelen = orig / high
        smooth = (orig / wavelen - low) / (high - low)
        mid = (1.0 - smooth) * inv / factor + smooth * inv
        inv = torch.where(wavelen < high_wavelen, inv,
                          torch.where(wavelen > low_wavelen, inv / factor, mid))
    return inv


def plain_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """rotate_half over the first 2*len(inv_freq) channels of each head.

    x: [T, heads, head_dim].  Pair (j, j + rd/2): (a cos - b sin, a sin + b cos)
    with angle = pos * inv_j (src/kernels/rope.cu:23-34).  The angle is formed in
    32-bit as the engine does (position and frequency both float32), then the
    sine and cosine are taken in x's dtype.
    """
    rd = 2 * inv_freq.numel()
    positions, inv_freq = positions.to(x.device), inv_freq.to(x.device)
    ang = (positions.to(torch.float32)[:, None] * inv_freq.to(torch.float32)[None, :]).to(x.dtype)
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., : rd // 2], x[..., rd // 2: rd]
    out = x.clone()
    out[..., : rd // 2] = a * cos - b * sin
    out[..., rd // 2: rd] = a * sin + b * cos
    return out


def plain_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                    window: Optional[int] = None, scale: Optional[float] = None) -> torch.Tensor:
    """Causal grouped-query softmax attention of one whole sequence.

    q: [T, nh, hd]; k, v: [T, nkv, hd].  Query head h reads kv head h // (nh/nkv);
    score = (q . k) * hd**-0.5, keys at positions <= the query's; softmax; P.V
    (src/kernels/paged_flash_attention.cu:60-61, 142-144, 120-190).  ``window``
    keeps only the last ``window`` keys (the query's own included).
    """
    T, nh, hd = q.shape
    nkv = k.shape[1]
    g = nh // nkv
    scale = hd ** -0.5 if scale is None else scale
    kk = k.repeat_interleave(g, dim=1)
    vv = v.repeat_interleave(g, dim=1)
    s = torch.einsum("thd,shd->hts", q, kk) * scale
    i = torch.arange(T, device=q.device)
    mask = i[None, :] <= i[:, None]
    if window is not None:
        mask &= i[None, :] > i[:, None] - window
    s = s.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hts,shd->thd", p, vv)


def plain_attention_tail(q_tail: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: Optional[int] = None,
                         rows_at_once: int = 512) -> torch.Tensor:
    """The same attention for the LAST ``len(q_tail)`` positions of a sequence only (the queries of a
    prompt portion, or a decode token, over all keys before them), a few hundred rows at a time so that
    long sequences fit in memory.  q_tail: [n, nh, hd]; k, v: [T, nkv, hd] -> [n, nh, hd]."""
    n, nh, hd = q_tail.shape
    T, nkv = k.shape[0], k.shape[1]
    g = nh // nkv
    start = T - n
    out = torch.empty_like(q_tail)
    key_pos = torch.arange(T, device=q_tail.device)
    for a in range(0, n, rows_at_once):
        b = min(n, a + rows_at_once)
        last = start + b                      # keys [0, last) can be seen by these rows
        qq = q_tail[a:b].view(b - a, nkv, g, hd)
        s = torch.einsum("tkgd,skd->kgts", qq, k[:last]) * hd ** -0.5
        qpos = start + torch.arange(a, b, device=q_tail.device)
        mask = key_pos[None, :last] <= qpos[:, None]
        if window is not None:
            mask &= key_pos[None, :last] > qpos[:, None] - window
        p = torch.softmax(s.masked_fill(~mask[None, None], float("-inf")), dim=-1)
        out[a:b] = torch.einsum("kgts,skd->tkgd", p, v[:last]).reshape(b - a, nh, hd)
    return out


def plain_swiglu(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """silu(g) * u with silu(g) = g / (1 + exp(-g)) (src/kernels/swiglu.cu:27-34)."""
    return g / (1.0 + torch.exp(-g)) * u


def plain_linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x W^T (+ b): weights are [out, in] (src/kernels/bf16_linear.cu:13-54;
    bias added once after the dot product, bf16_linear_bias.cu:44-50)."""
    y = x @ w.T
    return y if b is None else y + b


# --------------------------------------------------------------------------- whole model

def plain_layer(x, positions, W: Dict[str, torch.Tensor], i: int, c: dict, inv_freq,
                window: Optional[int] = None):
    """One decoder layer (src/core/engine.cpp:946-1024): pre-norm attention block
    with the output projection added to the residual stream, then pre-norm
    SwiGLU block likewise."""
    p = f"model.layers.{i}."
    T = x.shape[0]
    h = plain_rmsnorm(x, W[p + "input_layernorm.weight"], c["eps"])
    bq = W.get(p + "self_attn.q_proj.bias") if c["bias"] else None
    bk = W.get(p + "self_attn.k_proj.bias") if c["bias"] else None
    bv = W.get(p + "self_attn.v_proj.bias") if c["bias"] else None
    q = plain_linear(h, W[p + "self_attn.q_proj.weight"], bq).view(T, c["nh"], c["hd"])
    k = plain_linear(h, W[p + "self_attn.k_proj.weight"], bk).view(T, c["nkv"], c["hd"])
    v = plain_linear(h, W[p + "self_attn.v_proj.weight"], bv).view(T, c["nkv"], c["hd"])
    q = plain_rope(q, positions, inv_freq)
    k = plain_rope(k, positions, inv_freq)
    o = plain_attention(q, k, v, window=window).reshape(T, c["nh"] * c["hd"])
    x = x + plain_linear(o, W[p + "self_attn.o_proj.weight"])
    h = plain_rmsnorm(x, W[p + "post_attention_layernorm.weight"], c["eps"])
    a = plain_swiglu(plain_linear(h, W[p + "mlp.gate_proj.weight"]),
                     plain_linear(h, W[p + "mlp.up_proj.weight"]))
    return x + plain_linear(a, W[p + "mlp.down_proj.weight"])


def plain_logits(raw_config: dict, weights: Dict[str, torch.Tensor], ids: Sequence[int],
                 dtype=torch.float64, rows: Optional[Sequence[int]] = None, device=None) -> torch.Tensor:
    """Logits [T, V] at every position of one whole sequence
    (src/core/engine.cpp:921-1041: embedding, layers, final norm, lm_head; the
    head is the embedding table when tied, engine.cpp:668-670).  ``rows``: only
    these positions' logits (the whole sequence is computed all the same; the
    final norm and the head run on these rows).  ``device``: where torch does the
    arithmetic (the weights are copied there); the result comes back to the CPU."""
    c = plain_config(raw_config)
    W = {k: v.to(device=device, dtype=dtype) for k, v in weights.items()}
    x = plain_embedding(W["model.embed_tokens.weight"], ids)
    positions = torch.arange(len(ids))
    inv_freq = plain_inv_freq(c["hd"], c["theta"], c["scaling"], c["rd"])
    for i in range(c["L"]):
        x = plain_layer(x, positions, W, i, c, inv_freq)
    if rows is not None:
        x = x[torch.as_tensor(list(rows), dtype=torch.long, device=x.device)]
    x = plain_rmsnorm(x, W["model.norm.weight"], c["eps"])
    head = W["model.embed_tokens.weight"] if c["tie"] else W["lm_head.weight"]
    return plain_linear(x, head).cpu()


def plain_greedy(raw_config: dict, weights, prompt: Sequence[int], steps: int,
                 dtype=torch.float64) -> List[int]:
    """Greedy continuation, recomputing the whole sequence every step; the lowest
    index wins a tie."""
    ids = list(prompt)
    out = []
    for _ in range(steps):
        lg = plain_logits(raw_config, weights, ids, dtype)[-1]
        t = int(torch.argmax(lg))
        t = int((lg == lg[t]).nonzero()[0])
        out.append(t)
        ids.append(t)
    return out


def load_plain_weights(model_dir: str) -> Dict[str, torch.Tensor]:
    """Reads model.safetensors with the installed safetensors package (not with
    the product's reader)."""
    import os
    from safetensors.torch import load_file
    return load_file(os.path.join(model_dir, "model.safetensors"))
