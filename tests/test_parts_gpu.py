"""Each part alone against the plain functions, at sizes of its own; and a toy mixer
with per-request state, defined HERE, registered, built into a model and stepped
through the engine without a change to the package."""
from dataclasses import dataclass

import pytest
import torch

from blackwellllm_b200.kernels import ops
from plain_model import (plain_attention, plain_inv_freq, plain_linear, plain_rmsnorm, plain_rope, plain_swiglu)

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def make_batch(cache, segments, want_all=True):
    """segments: [(rid, n_tokens)]: grows the requests in ``cache`` and packs a batch."""
    from batch_packer import pack_batch
    from blackwellllm_b200.engine.batch import BatchBuilder
    segs, rows, t0 = [], [], 0
    for rid, n in segments:
        if not cache.has(rid):
            cache.add_request(rid)
        start = cache.append(rid, n)
        segs.append((rid, [0] * n, start, start + n, cache.slot(rid)))
        rows += list(range(t0, t0 + n))
        t0 += n
    block_rows = {g: [cache.block_table(rid, g) for rid, _ in segments] for g in range(len(cache.groups))}
    return pack_batch(BatchBuilder(DEV), segs, rows if want_all else [], block_rows)


TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from blackwellllm_b200.config.specs import RMSNormSpec
    from blackwellllm_b200.parts import BuildContext, build_norm
    H = 200
    norm = build_norm(RMSNormSpec(eps=3e-4), H, BuildContext(DEV, dtype))
    assert [p.name for p in norm.param_specs()] == ["weight"] and norm.param_specs()[0].shape == (H,)
    w = rnd(H, seed=1).to(dtype)
    norm.bind({"weight": w.to(DEV)})
    x = rnd(9, H, seed=2, scale=4.0)
    out = norm.forward(x.to(DEV))
    ref = plain_rmsnorm(x.double(), w.double(), 3e-4)
    assert out.dtype == dtype
    assert float((out.double().cpu() - ref).abs().max()) <= TOL[dtype] * float(ref.abs().max())


def test_inv_freq_table_all_three_bands():
    from blackwellllm_b200.config.specs import Llama3RopeScaling
    from blackwellllm_b200.parts.rope import rotary_inv_freq
    sc = Llama3RopeScaling(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=8192)
    ours = rotary_inv_freq(500000.0, 128, sc).double()
    ref = plain_inv_freq(128, 500000.0, (8.0, 1.0, 4.0, 8192))
    assert float(((ours - ref) / ref).abs().max()) < 1e-6
    plain = plain_inv_freq(128, 500000.0, None)
    ratio = ref / plain
    assert bool((ratio == 1).any()) and bool(((ratio - 0.125).abs() < 1e-12).any())
    assert bool(((ratio > 0.126) & (ratio < 0.999)).any())          # the interpolated band is hit too


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rotary_dim,scaling", [(48, None), (24, None), (48, (4.0, 1.0, 4.0, 64))])
def test_rotary_encoding_and_append(dtype, rotary_dim, scaling):
    from blackwellllm_b200.cache.manager import CacheManager
    from blackwellllm_b200.config.specs import Llama3RopeScaling, RopeSpec
    from blackwellllm_b200.parts import BuildContext, PagedKVRequest, build_position
    nh, nkv, hd, page = 6, 2, 48, 8
    sc = None if scaling is None else Llama3RopeScaling(*scaling)
    pos_enc = build_position(RopeSpec(theta=10000.0, rotary_dim=rotary_dim, scaling=sc), hd, BuildContext(DEV, dtype))
    cache = CacheManager([PagedKVRequest(nkv, hd)], page, 700, 4, dtype=dtype, device=DEV)
    # request "far" already holds 5000 tokens, so positions are large; request "new" starts at 0
    cache.add_request("far")
    cache.append("far", 5000)
    batch = make_batch(cache, [("far", 19), ("new", 30)])
    T = 49
    qkv = rnd(T, (nh + 2 * nkv) * hd, seed=3)
    q = pos_enc.rotate_append(qkv.to(DEV), batch, cache.views[0], nh, nkv, hd)
    positions = torch.tensor(list(range(5000, 5019)) + list(range(30)))
    inv = plain_inv_freq(hd, 10000.0, scaling, rotary_dim=rotary_dim)
    x = qkv.double().view(T, nh + 2 * nkv, hd)
    q_ref = plain_rope(x[:, :nh], positions, inv).reshape(T, nh * hd)
    k_ref = plain_rope(x[:, nh:nh + nkv], positions, inv)
    v_ref = x[:, nh + nkv:]
    tol = 2e-6 if dtype == torch.float32 else 2 ** -8
    assert float((q.double().cpu() - q_ref).abs().max()) <= tol * float(q_ref.abs().max())
    view = cache.views[0]
    for t in range(T):
        rid = "far" if t < 19 else "new"
        p = int(positions[t])
        pg = cache.block_table(rid, 0)[p // page]
        k_got = view.k_pages[pg, :, p % page].double().cpu()
        v_got = view.v_pages[pg, :, p % page].double().cpu()
        assert float((k_got - k_ref[t]).abs().max()) <= tol * float(k_ref.abs().max())
        assert float((v_got - v_ref[t]).abs().max()) <= tol * float(v_ref.abs().max())


@pytest.mark.parametrize("lens", [(1, 2), (19, 30), (150, 171)])
@pytest.mark.parametrize("rotary_dim,bias", [(48, True), (24, False)])
def test_rotary_encoding_inside_the_projection(lens, rotary_dim, bias):
    """bfloat16: projection, rotation and append in one kernel (few tokens with K splits summed
    inside the kernel, more with the second kernel, many in the other orientation) against
    plain projection + plain rotation."""
    from blackwellllm_b200.cache.manager import CacheManager
    from blackwellllm_b200.config.specs import RopeSpec
    from blackwellllm_b200.parts import BuildContext, PagedKVRequest, build_position
    nh, nkv, hd, page, K = 6, 2, 48, 8, 1096
    dtype = torch.bfloat16
    pos_enc = build_position(RopeSpec(theta=10000.0, rotary_dim=rotary_dim, scaling=None), hd, BuildContext(DEV, dtype))
    cache = CacheManager([PagedKVRequest(nkv, hd)], page, 700, 4, dtype=dtype, device=DEV)
    cache.add_request("far")
    cache.append("far", 5000)
    batch = make_batch(cache, [("far", lens[0]), ("new", lens[1])])
    T = sum(lens)
    w = rnd((nh + 2 * nkv) * hd, K, seed=5, scale=0.05).to(dtype)
    b = rnd((nh + 2 * nkv) * hd, seed=6, scale=0.5).to(dtype) if bias else None
    x = rnd(T, K, seed=7).to(dtype)
    project = pos_enc.fuse_projection(w.to(DEV), None if b is None else b.to(DEV), nh, nkv, hd)
    assert project is not None
    q = project(x.to(DEV), batch, cache.views[0], True)
    positions = torch.tensor(list(range(5000, 5000 + lens[0])) + list(range(lens[1])))
    inv = plain_inv_freq(hd, 10000.0, None, rotary_dim=rotary_dim)
    qkv = x.double() @ w.double().T + (0 if b is None else b.double())
    qkv = qkv.view(T, nh + 2 * nkv, hd)
    q_ref = plain_rope(qkv[:, :nh], positions, inv).reshape(T, nh * hd)
    k_ref = plain_rope(qkv[:, nh:nh + nkv], positions, inv)
    v_ref = qkv[:, nh + nkv:]
    tol = 2 ** -7    # bfloat16 results of float32 sums over 1096 products
    assert float((q.double().cpu() - q_ref).abs().max()) <= tol * float(q_ref.abs().max())
    view = cache.views[0]
    kp, vp = view.k_pages.double().cpu(), view.v_pages.double().cpu()
    for t in range(T):
        rid = "far" if t < lens[0] else "new"
        p_ = int(positions[t])
        pg = cache.block_table(rid, 0)[p_ // page]
        assert float((kp[pg, :, p_ % page] - k_ref[t]).abs().max()) <= tol * float(k_ref.abs().max())
        assert float((vp[pg, :, p_ % page] - v_ref[t]).abs().max()) <= tol * float(v_ref.abs().max())
    assert ops_status() == 0


def ops_status():
    from blackwellllm_b200.kernels import ops
    return ops.gemm_tc_status()


def attention_weights(H, nh, nkv, hd, bias, dtype, seed):
    t = {"q_proj.weight": rnd(nh * hd, H, seed=seed, scale=0.1), "k_proj.weight": rnd(nkv * hd, H, seed=seed + 1, scale=0.1),
         "v_proj.weight": rnd(nkv * hd, H, seed=seed + 2, scale=0.1), "o_proj.weight": rnd(H, nh * hd, seed=seed + 3, scale=0.1)}
    if bias:
        t.update({"q_proj.bias": rnd(nh * hd, seed=seed + 4, scale=0.3), "k_proj.bias": rnd(nkv * hd, seed=seed + 5, scale=0.3),
                  "v_proj.bias": rnd(nkv * hd, seed=seed + 6, scale=0.3)})
    return {k: v.to(dtype) for k, v in t.items()}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("bias,window", [(False, None), (True, None), (True, 20)])
def test_attention_mixer_alone(dtype, bias, window):
    from blackwellllm_b200.cache.manager import CacheManager
    from blackwellllm_b200.config.specs import AttentionSpec, RopeSpec
    from blackwellllm_b200.parts import BuildContext, build_mixer
    H, nh, nkv, hd, page = 72, 6, 3, 16, 8
    spec = AttentionSpec(nh, nkv, hd, bias, RopeSpec(1e4, hd), window=window)
    mixer = build_mixer(spec, H, BuildContext(DEV, dtype))
    names = {p.name for p in mixer.param_specs()}
    assert ("q_proj.bias" in names) == bias
    W = attention_weights(H, nh, nkv, hd, bias, dtype, 10)
    mixer.bind({k: v.to(DEV) for k, v in W.items()})
    cache = CacheManager([mixer.cache_request()], page, 64, 4, dtype=dtype, device=DEV)
    lens = {"a": 45, "b": 70}
    xs = {r: rnd(n, H, seed=len(r) + n).to(dtype) for r, n in lens.items()}

    def plain(x):
        xd = x.double()
        T = x.shape[0]
        Wd = {k: v.double() for k, v in W.items()}
        q = plain_linear(xd, Wd["q_proj.weight"], Wd.get("q_proj.bias")).view(T, nh, hd)
        k = plain_linear(xd, Wd["k_proj.weight"], Wd.get("k_proj.bias")).view(T, nkv, hd)
        v = plain_linear(xd, Wd["v_proj.weight"], Wd.get("v_proj.bias")).view(T, nkv, hd)
        inv = plain_inv_freq(hd, 1e4, None)
        pos = torch.arange(T)
        o = plain_attention(plain_rope(q, pos, inv), plain_rope(k, pos, inv), v, window=window)
        return plain_linear(o.reshape(T, nh * hd), Wd["o_proj.weight"])

    # first step: most of "a" and a part of "b"; second step: the rest of both, "a" one token short, then its last
    cuts = [[("a", 40), ("b", 33)], [("a", 4), ("b", 37)], [("a", 1)]]
    done = {"a": 0, "b": 0}
    got = {r: [] for r in lens}
    for step in cuts:
        batch = make_batch(cache, step)
        x = torch.cat([xs[r][done[r]:done[r] + n] for r, n in step]).to(DEV)
        residual = torch.zeros(x.shape[0], H, device=DEV)
        mixer.forward(x, residual, batch, cache.views[0], True)
        ops.resolve_pending()   # a few tokens: the output projection leaves its sum to the stream's next reader
        at = 0
        for r, n in step:
            got[r].append(residual[at:at + n].double().cpu())
            at += n
            done[r] += n
            cache.release_passed(r)
    for r in lens:
        ref = plain(xs[r])
        out = torch.cat(got[r])
        assert float((out - ref).abs().max()) <= TOL[dtype] * float(ref.abs().max()), r
    if window:
        assert -1 in cache.block_table("b", 0)    # pages behind the window went back to the pool


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part_and_block(dtype):
    from blackwellllm_b200.cache.manager import CacheManager
    from blackwellllm_b200.config.specs import AttentionSpec, LayerSpec, RMSNormSpec, RopeSpec, SwiGLUSpec
    from blackwellllm_b200.parts import BuildContext, build_block, build_ffn
    H, I = 72, 200
    ctx = BuildContext(DEV, dtype)
    ffn = build_ffn(SwiGLUSpec(I), H, ctx)
    Wf = {"gate_proj.weight": rnd(I, H, seed=1, scale=0.1).to(dtype), "up_proj.weight": rnd(I, H, seed=2, scale=0.1).to(dtype),
          "down_proj.weight": rnd(H, I, seed=3, scale=0.1).to(dtype)}
    ffn.bind({k: v.to(DEV) for k, v in Wf.items()})
    x = rnd(11, H, seed=4).to(dtype)
    res = torch.ones(11, H, device=DEV)
    ffn.forward(x.to(DEV), res, None)
    assert (ops.pending_target() is res) == (dtype == torch.bfloat16)   # 11 tokens: the down projection's sum is left open
    ops.resolve_pending()
    xd = x.double()
    ref = 1.0 + plain_linear(plain_swiglu(plain_linear(xd, Wf["gate_proj.weight"].double()),
                                          plain_linear(xd, Wf["up_proj.weight"].double())), Wf["down_proj.weight"].double())
    assert float((res.double().cpu() - ref).abs().max()) <= TOL[dtype] * float(ref.abs().max())

    # the whole pre-norm block: x += attn(norm(x)); x += ffn(norm(x))
    nh, nkv, hd = 6, 3, 16
    layer = LayerSpec(AttentionSpec(nh, nkv, hd, True, RopeSpec(1e4, hd)), SwiGLUSpec(I), RMSNormSpec(1e-5), RMSNormSpec(1e-5))
    block = build_block(layer, H, ctx)
    Wa = attention_weights(H, nh, nkv, hd, True, dtype, 20)
    g1, g2 = (1 + rnd(H, seed=30, scale=0.1)).to(dtype), (1 + rnd(H, seed=31, scale=0.1)).to(dtype)
    tensors = {"self_attn." + k: v for k, v in Wa.items()}
    tensors.update({"mlp." + k: v for k, v in Wf.items()})
    tensors.update({"input_layernorm.weight": g1, "post_attention_layernorm.weight": g2})
    assert {p.name for p in block.param_specs()} == set(tensors)
    block.bind({k: v.to(DEV) for k, v in tensors.items()})
    cache = CacheManager([block.mixer.cache_request()], 8, 16, 2, dtype=dtype, device=DEV)
    T = 37
    h0 = rnd(T, H, seed=5)
    h = h0.clone().to(DEV)
    block.forward(h, make_batch(cache, [("a", T)]), cache.views[0], True)
    ops.resolve_pending()
    hd_ = h0.double()
    n1 = plain_rmsnorm(hd_, g1.double(), 1e-5)
    Wd = {k: v.double() for k, v in Wa.items()}
    pos, inv = torch.arange(T), plain_inv_freq(hd, 1e4, None)
    q = plain_rope(plain_linear(n1, Wd["q_proj.weight"], Wd["q_proj.bias"]).view(T, nh, hd), pos, inv)
    k = plain_rope(plain_linear(n1, Wd["k_proj.weight"], Wd["k_proj.bias"]).view(T, nkv, hd), pos, inv)
    v = plain_linear(n1, Wd["v_proj.weight"], Wd["v_proj.bias"]).view(T, nkv, hd)
    hd_ = hd_ + plain_linear(plain_attention(q, k, v).reshape(T, nh * hd), Wd["o_proj.weight"])
    n2 = plain_rmsnorm(hd_, g2.double(), 1e-5)
    hd_ = hd_ + plain_linear(plain_swiglu(plain_linear(n2, Wf["gate_proj.weight"].double()),
                                          plain_linear(n2, Wf["up_proj.weight"].double())), Wf["down_proj.weight"].double())
    assert float((h.double().cpu() - hd_).abs().max()) <= TOL[dtype] * float(hd_.abs().max())


@dataclass(frozen=True)
class ToyScaleNormSpec:
    kind: str = "toy_scalenorm"


def register_toy_scalenorm():
    from blackwellllm_b200.parts import Norm, ParamSpec, register_norm

    class ToyScaleNorm(Norm):
        """y = x * w / (1 + mean |x|), computed with torch on the stream itself: it knows nothing of sums that a
        product left open, so the block has to make them before it calls this."""
        def __init__(self, spec, hidden_size, ctx):
            self.hidden_size, self.ctx, self.weight = hidden_size, ctx, None

        def param_specs(self):
            return [ParamSpec("weight", (self.hidden_size,), role="gain", init="ones")]

        def bind(self, tensors):
            self.weight = tensors["weight"].float()

        def forward(self, x, rows=None):
            if rows is not None:
                x = x[rows.long()]
            return (x * self.weight / (1 + x.abs().mean(-1, keepdim=True))).to(self.ctx.dtype)

    register_norm("toy_scalenorm", ToyScaleNorm)


@pytest.mark.parametrize("norm", ["rmsnorm", "toy_scalenorm"])
@pytest.mark.parametrize("T", [1, 5, 16, 40, 128, 129])
def test_block_on_few_tokens_where_products_leave_their_sums_open(norm, T):
    """Up to ``ops.DEFER_MAX_TOKENS`` tokens the output and the down projection leave the sums of their K splits to the
    next reader of the stream: an RMSNorm adds them while it normalises, before any other norm the block adds them itself."""
    from blackwellllm_b200.cache.manager import CacheManager
    from blackwellllm_b200.config.specs import AttentionSpec, LayerSpec, RMSNormSpec, RopeSpec, SwiGLUSpec
    from blackwellllm_b200.parts import BuildContext, build_block
    register_toy_scalenorm()
    dtype = torch.bfloat16
    H, I, nh, nkv, hd = 136, 208, 6, 3, 16
    ctx = BuildContext(DEV, dtype)
    nspec = RMSNormSpec(1e-5) if norm == "rmsnorm" else ToyScaleNormSpec()
    block = build_block(LayerSpec(AttentionSpec(nh, nkv, hd, True, RopeSpec(1e4, hd)), SwiGLUSpec(I), nspec, nspec), H, ctx)
    Wa = attention_weights(H, nh, nkv, hd, True, dtype, 20)
    Wf = {"gate_proj.weight": rnd(I, H, seed=1, scale=0.1).to(dtype), "up_proj.weight": rnd(I, H, seed=2, scale=0.1).to(dtype),
          "down_proj.weight": rnd(H, I, seed=3, scale=0.1).to(dtype)}
    g1, g2 = (1 + rnd(H, seed=30, scale=0.1)).to(dtype), (1 + rnd(H, seed=31, scale=0.1)).to(dtype)
    tensors = {"self_attn." + k: v for k, v in Wa.items()}
    tensors.update({"mlp." + k: v for k, v in Wf.items()})
    tensors.update({"input_layernorm.weight": g1, "post_attention_layernorm.weight": g2})
    block.bind({k: v.to(DEV) for k, v in tensors.items()})
    cache = CacheManager([block.mixer.cache_request()], 8, 20, 2, dtype=dtype, device=DEV)
    h0 = rnd(T, H, seed=5)
    h = h0.clone().to(DEV)
    block.forward(h, make_batch(cache, [("a", T)]), cache.views[0], True)
    assert ops.DEFER_MAX_TOKENS == 128
    assert (ops.pending_target() is h) == (T <= 128)   # the down projection's sum is still open when the block returns
    ops.resolve_pending()

    def plain_norm(x, g):
        if norm == "rmsnorm":
            return plain_rmsnorm(x, g.double(), 1e-5)
        return x * g.double() / (1 + x.abs().mean(-1, keepdim=True))

    x = h0.double()
    n1 = plain_norm(x, g1)
    Wd = {k: v.double() for k, v in Wa.items()}
    pos, inv = torch.arange(T), plain_inv_freq(hd, 1e4, None)
    q = plain_rope(plain_linear(n1, Wd["q_proj.weight"], Wd["q_proj.bias"]).view(T, nh, hd), pos, inv)
    k = plain_rope(plain_linear(n1, Wd["k_proj.weight"], Wd["k_proj.bias"]).view(T, nkv, hd), pos, inv)
    v = plain_linear(n1, Wd["v_proj.weight"], Wd["v_proj.bias"]).view(T, nkv, hd)
    x = x + plain_linear(plain_attention(q, k, v).reshape(T, nh * hd), Wd["o_proj.weight"])
    n2 = plain_norm(x, g2)
    x = x + plain_linear(plain_swiglu(plain_linear(n2, Wf["gate_proj.weight"].double()),
                                      plain_linear(n2, Wf["up_proj.weight"].double())), Wf["down_proj.weight"].double())
    assert float((h.double().cpu() - x).abs().max()) <= TOL[dtype] * float(x.abs().max())


# ---------------------------------------------------------------------------------------------
# A toy mixer with state of its own: an exponential moving average of a projection of the
# tokens, one state vector per request.  Everything it needs is defined in this file.

@dataclass(frozen=True)
class ToyEmaSpec:
    decay: float
    kind: str = "toy_ema"


def register_toy():
    from blackwellllm_b200.config import ModelConfig, ScheduleEntry, register_architecture
    from blackwellllm_b200.config.specs import AttentionSpec, LayerSpec, RMSNormSpec, RopeSpec, SwiGLUSpec
    from blackwellllm_b200.parts import FixedStateRequest, Mixer, ParamSpec, register_mixer

    class ToyEma(Mixer):
        graph_safe = False   # it loops on the host: the engine must not capture it in a CUDA graph

        def __init__(self, spec, hidden_size, ctx):
            self.decay, self.H, self.ctx = spec.decay, hidden_size, ctx

        def cache_request(self):
            return FixedStateRequest((self.H,), torch.float32)

        def param_specs(self):
            return [ParamSpec("in_proj.weight", (self.H, self.H))]

        def bind(self, tensors):
            self.w = tensors["in_proj.weight"].float()

        def forward(self, x, residual, batch, cache, owns_cache=True):
            y = x.float() @ self.w.T            # a toy: plain tensor ops, token by token
            cu = [0]
            for n in batch.h_q_len:
                cu.append(cu[-1] + n)
            for r, slot in enumerate(batch.h_slots):
                s = cache.state[slot]
                for t in range(cu[r], cu[r + 1]):
                    s = self.decay * s + (1 - self.decay) * y[t]
                    residual[t] += s
                cache.state[slot] = s

    register_mixer("toy_ema", ToyEma)

    def parse(raw):
        H = raw["hidden_size"]
        toy = LayerSpec(ToyEmaSpec(raw["decay"]), None, RMSNormSpec(raw["eps"]), None, mixer_prefix="ema.")
        att = LayerSpec(AttentionSpec(raw["heads"], raw["kv_heads"], raw["head_dim"], False, RopeSpec(1e4, raw["head_dim"])),
                        SwiGLUSpec(raw["inter"]), RMSNormSpec(raw["eps"]), RMSNormSpec(raw["eps"]))
        return ModelConfig(architecture="ToyForCausalLM", hidden_size=H, vocab_size=raw["vocab_size"],
                           layers=(toy, att), schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0)),
                           final_norm=RMSNormSpec(raw["eps"]), tie_word_embeddings=True, max_position_embeddings=0, raw=dict(raw))

    register_architecture("ToyForCausalLM", parse)


def test_toy_mixer_with_state_registers_builds_and_steps():
    from blackwellllm_b200 import Engine, StepEntry
    from blackwellllm_b200.weights.random_init import model_param_specs, random_tensors
    register_toy()
    raw = {"architectures": ["ToyForCausalLM"], "hidden_size": 48, "vocab_size": 90, "decay": 0.8, "eps": 1e-5,
           "heads": 3, "kv_heads": 1, "head_dim": 16, "inter": 100}
    specs = model_param_specs(raw)
    assert "model.layers.0.ema.in_proj.weight" in specs and "model.layers.1.self_attn.q_proj.weight" in specs
    W = random_tensors(specs, seed=4, std=0.2, dtype=torch.float32)
    eng = Engine.from_tensors(raw, W, dtype="float32", page_size=8, max_tokens=128, max_requests=2)
    # layer 0 runs twice (schedule entries 0 and 2) with separate state; entry 1 is attention
    assert len(eng.cache.groups) == 1 and sum(v is not None for v in eng.cache.views) == 3

    def plain(ids):
        Wd = {k: v.double() for k, v in W.items()}
        x = Wd["model.embed_tokens.weight"][torch.tensor(ids)]
        T = len(ids)

        def ema(x):
            y = plain_rmsnorm(x, Wd["model.layers.0.input_layernorm.weight"], 1e-5) @ Wd["model.layers.0.ema.in_proj.weight"].T
            s, out = torch.zeros(48, dtype=torch.float64), x.clone()
            for t in range(T):
                s = 0.8 * s + 0.2 * y[t]
                out[t] += s
            return out
        x = ema(x)
        p = "model.layers.1."
        n1 = plain_rmsnorm(x, Wd[p + "input_layernorm.weight"], 1e-5)
        pos, inv = torch.arange(T), plain_inv_freq(16, 1e4, None)
        q = plain_rope(plain_linear(n1, Wd[p + "self_attn.q_proj.weight"]).view(T, 3, 16), pos, inv)
        k = plain_rope(plain_linear(n1, Wd[p + "self_attn.k_proj.weight"]).view(T, 1, 16), pos, inv)
        v = plain_linear(n1, Wd[p + "self_attn.v_proj.weight"]).view(T, 1, 16)
        x = x + plain_linear(plain_attention(q, k, v).reshape(T, 48), Wd[p + "self_attn.o_proj.weight"])
        n2 = plain_rmsnorm(x, Wd[p + "post_attention_layernorm.weight"], 1e-5)
        x = x + plain_linear(plain_swiglu(plain_linear(n2, Wd[p + "mlp.gate_proj.weight"]),
                                          plain_linear(n2, Wd[p + "mlp.up_proj.weight"])), Wd[p + "mlp.down_proj.weight"])
        x = ema(x)
        return plain_linear(plain_rmsnorm(x, Wd["model.norm.weight"], 1e-5), Wd["model.embed_tokens.weight"])

    g = torch.Generator().manual_seed(0)
    a = torch.randint(0, 90, (30,), generator=g).tolist()
    b = torch.randint(0, 90, (21,), generator=g).tolist()
    c = torch.randint(0, 90, (17,), generator=g).tolist()
    ref = {"a": plain(a), "b": plain(b), "c": plain(c)}
    got = {"a": [], "b": [], "c": []}

    def run(entries):
        out = eng.step([StepEntry(r, t, list(range(len(t)))) for r, t in entries]).double().cpu()
        at = 0
        for r, t in entries:
            got[r].append(out[at:at + len(t)])
            at += len(t)

    run([("a", a[:13])])
    run([("a", a[13:14]), ("b", b[:9])])          # a decodes beside a portion of b
    run([("b", b[9:]), ("a", a[14:])])
    eng.end_request("a")
    run([("c", c[:2])])                           # c takes over a's slot: its state must start at zero
    run([("c", c[2:])])
    for r in got:
        out = torch.cat(got[r])
        assert float((out - ref[r]).abs().max()) <= 1e-4 * float(ref[r].abs().max()), r


# ---------------------------------------------------------------------------------------------
# A toy feed-forward with routing (each token goes to the expert its router scores highest) and a
# toy position encoding (a sinusoid of the position added to queries and keys), both defined here,
# inside a model whose second layer reads the first layer's cache instead of keeping one.

@dataclass(frozen=True)
class ToyRoutedSpec:
    experts: int
    kind: str = "toy_routed"


@dataclass(frozen=True)
class ToyAddPosSpec:
    period: float
    kind: str = "toy_addpos"


def toy_add_pos(x, positions, period):
    """x [T, heads, hd] + sin(pos / period + channel)."""
    hd = x.shape[-1]
    ang = positions.to(x.dtype)[:, None] / period + torch.arange(hd, dtype=x.dtype, device=x.device)[None, :]
    return x + torch.sin(ang)[:, None, :]


def register_toy_routed():
    from blackwellllm_b200.config import ModelConfig, ScheduleEntry, register_architecture
    from blackwellllm_b200.config.specs import AttentionSpec, LayerSpec, RMSNormSpec
    from blackwellllm_b200.parts import FeedForward, ParamSpec, PositionEncoding, register_ffn, register_position

    class ToyRouted(FeedForward):
        def __init__(self, spec, hidden_size, ctx):
            self.E, self.H = spec.experts, hidden_size

        def param_specs(self):
            return [ParamSpec("router.weight", (self.E, self.H))] + \
                   [ParamSpec(f"experts.{e}.weight", (self.H, self.H)) for e in range(self.E)]

        def bind(self, tensors):
            self.router = tensors["router.weight"].float()
            self.experts = torch.stack([tensors[f"experts.{e}.weight"].float() for e in range(self.E)])

        def forward(self, x, residual, batch):
            xf = x.float()
            choice = (xf @ self.router.T).argmax(dim=1)                   # router logits in 32-bit
            y = torch.einsum("th,toh->to", xf, self.experts[choice])
            residual += torch.relu(y)

    class ToyAddPos(PositionEncoding):
        def __init__(self, spec, head_dim, ctx):
            self.period = spec.period

        def rotate_append(self, qkv, batch, cache, nh, nkv, hd, append=True):
            T = qkv.shape[0]
            x = qkv.float().view(T, nh + 2 * nkv, hd)
            pos = batch.positions.long()
            q = toy_add_pos(x[:, :nh], pos, self.period)
            if append:
                k = toy_add_pos(x[:, nh:nh + nkv], pos, self.period)
                ps = cache.k_pages.shape[2]
                pages = batch.block_tables[cache.group][batch.req_of_token.long(), pos // ps].long()
                cache.k_pages[pages, :, pos % ps] = k.to(cache.k_pages.dtype)
                cache.v_pages[pages, :, pos % ps] = x[:, nh + nkv:].to(cache.v_pages.dtype)
            return q.reshape(T, nh * hd).to(cache.k_pages.dtype)

    register_ffn("toy_routed", ToyRouted)
    register_position("toy_addpos", ToyAddPos)

    def parse(raw):
        att = AttentionSpec(raw["heads"], raw["kv_heads"], raw["head_dim"], False, ToyAddPosSpec(raw["period"]))
        layer = LayerSpec(att, ToyRoutedSpec(raw["experts"]), RMSNormSpec(raw["eps"]), RMSNormSpec(raw["eps"]))
        # the third entry runs layer 0 again on the keys and values that entry 0 wrote
        return ModelConfig(architecture="ToyRoutedForCausalLM", hidden_size=raw["hidden_size"],
                           vocab_size=raw["vocab_size"], layers=(layer, layer),
                           schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0, cache_of=0)),
                           final_norm=RMSNormSpec(raw["eps"]), tie_word_embeddings=True,
                           max_position_embeddings=0, raw=dict(raw))

    register_architecture("ToyRoutedForCausalLM", parse)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_routed_ffn_and_toy_position_encoding(dtype):
    from blackwellllm_b200 import Engine, StepEntry
    from blackwellllm_b200.weights.random_init import model_param_specs, random_tensors
    register_toy_routed()
    raw = {"architectures": ["ToyRoutedForCausalLM"], "hidden_size": 40, "vocab_size": 70, "eps": 1e-5,
           "heads": 5, "kv_heads": 5, "head_dim": 16, "experts": 3, "period": 7.0}
    specs = model_param_specs(raw)
    assert "model.layers.1.mlp.experts.2.weight" in specs and "model.layers.0.mlp.router.weight" in specs
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    W = random_tensors(specs, seed=9, std=0.3, dtype=tdt)
    eng = Engine.from_tensors(raw, W, dtype=dtype, page_size=8, max_tokens=128, max_requests=2)
    assert sum(v is not None for v in eng.cache.views) == 2     # entries 0 and 1 own a cache, entry 2 reads entry 0's

    def plain(ids):
        Wd = {k: v.double() for k, v in W.items()}
        T = len(ids)
        x = Wd["model.embed_tokens.weight"][torch.tensor(ids)]
        pos = torch.arange(T)
        kept = {}

        def layer(x, i, read_from=None):
            p = f"model.layers.{i}."
            n1 = plain_rmsnorm(x, Wd[p + "input_layernorm.weight"], 1e-5)
            q = toy_add_pos(plain_linear(n1, Wd[p + "self_attn.q_proj.weight"]).view(T, 5, 16), pos, 7.0)
            if read_from is None:
                k = toy_add_pos(plain_linear(n1, Wd[p + "self_attn.k_proj.weight"]).view(T, 5, 16), pos, 7.0)
                v = plain_linear(n1, Wd[p + "self_attn.v_proj.weight"]).view(T, 5, 16)
                if dtype == "bfloat16":   # the cache holds bfloat16
                    k, v = k.bfloat16().double(), v.bfloat16().double()
                kept[i] = (k, v)
            else:
                k, v = kept[read_from]
            x = x + plain_linear(plain_attention(q, k, v).reshape(T, 80), Wd[p + "self_attn.o_proj.weight"])
            n2 = plain_rmsnorm(x, Wd[p + "post_attention_layernorm.weight"], 1e-5)
            choice = (n2 @ Wd[p + "mlp.router.weight"].T).argmax(dim=1)
            ex = torch.stack([Wd[p + f"mlp.experts.{e}.weight"] for e in range(3)])
            return x + torch.relu(torch.einsum("th,toh->to", n2, ex[choice])), choice
        x, c0 = layer(x, 0)
        x, c1 = layer(x, 1)
        x, c2 = layer(x, 0, read_from=0)
        assert len(set(c0.tolist()) | set(c1.tolist()) | set(c2.tolist())) == 3    # every expert is used
        return plain_linear(plain_rmsnorm(x, Wd["model.norm.weight"], 1e-5), Wd["model.embed_tokens.weight"])

    g = torch.Generator().manual_seed(1)
    a = torch.randint(0, 70, (29,), generator=g).tolist()
    b = torch.randint(0, 70, (12,), generator=g).tolist()
    ref = {"a": plain(a), "b": plain(b)}
    got = {"a": [], "b": []}

    def run(entries):
        out = eng.step([StepEntry(r, t, list(range(len(t)))) for r, t in entries]).double().cpu()
        at = 0
        for r, t in entries:
            got[r].append(out[at:at + len(t)])
            at += len(t)

    run([("a", a[:11])])
    run([("a", a[11:12]), ("b", b[:7])])
    run([("b", b[7:]), ("a", a[12:27])])
    run([("a", a[27:28])])
    run([("a", a[28:])])
    tol = 1e-4 if dtype == "float32" else 4e-2
    for r in got:
        out = torch.cat(got[r])
        if dtype == "float32":
            assert float((out - ref[r]).abs().max()) <= tol * float(ref[r].abs().max()), r
        else:
            # a token whose two best router scores nearly tie may take the other expert in bfloat16:
            # compare the rows where the engine's rounding cannot have flipped a choice
            close = (out - ref[r]).abs().amax(dim=1) <= tol * float(ref[r].abs().max())
            assert float(close.double().mean()) >= 0.8, r


# ---------------------------------------------------------------------------------------------
# A mixer with state of its own that CAN be captured (device work only): decode steps of a model
# with it run from the CUDA graph, and the step that records the graph must advance the state once.

@dataclass(frozen=True)
class ToyCountSpec:
    kind: str = "toy_count"


def register_toy_count():
    from blackwellllm_b200.config import ModelConfig, ScheduleEntry, register_architecture
    from blackwellllm_b200.config.specs import LayerSpec, RMSNormSpec
    from blackwellllm_b200.parts import FixedStateRequest, Mixer, register_mixer

    class ToyCount(Mixer):
        """state[slot] += 1 per token; adds the request's count so far to every channel of the token."""
        graph_safe = True

        def __init__(self, spec, hidden_size, ctx):
            self.H = hidden_size

        def cache_request(self):
            return FixedStateRequest((1,), torch.float32)

        def forward(self, x, residual, batch, cache, owns_cache=True):
            slots = batch.state_slot.long()[batch.req_of_token.long()]           # [T], no host round trip
            before = cache.state[slots, 0]
            rank = (torch.arange(batch.T, device=x.device) - batch.cu_q.long()[batch.req_of_token.long()]).float()
            residual += (before + rank + 1.0)[:, None]
            cache.state.index_put_((slots, torch.zeros_like(slots)), torch.ones_like(before), accumulate=True)

    register_mixer("toy_count", ToyCount)

    def parse(raw):
        layer = LayerSpec(ToyCountSpec(), None, RMSNormSpec(1e-5), None, mixer_prefix="count.")
        return ModelConfig(architecture="ToyCountForCausalLM", hidden_size=raw["hidden_size"], vocab_size=raw["vocab_size"],
                           layers=(layer,), schedule=(ScheduleEntry(0),), final_norm=RMSNormSpec(1e-5),
                           tie_word_embeddings=True, max_position_embeddings=0, raw=dict(raw))

    register_architecture("ToyCountForCausalLM", parse)


def test_graph_safe_stateful_mixer_is_advanced_once_by_the_step_that_records_the_graph():
    from blackwellllm_b200 import Engine, StepEntry
    from blackwellllm_b200.weights.random_init import model_param_specs, random_tensors
    register_toy_count()
    raw = {"architectures": ["ToyCountForCausalLM"], "hidden_size": 32, "vocab_size": 50}
    W = random_tensors(model_param_specs(raw), seed=2, std=0.3, dtype=torch.float32)

    def run(graphs):
        eng = Engine.from_tensors(raw, W, dtype="float32", page_size=8, max_tokens=64, max_requests=2, cuda_graphs=graphs,
                                  graph_after=1)
        outs = [eng.step([StepEntry("a", [1, 2, 3], [2]), StepEntry("b", [4], [0])]).clone()]
        for t in (5, 6, 7):                       # decode-only steps of batch size 2: recorded at the first, replayed after
            outs.append(eng.step([StepEntry("a", [t], [0]), StepEntry("b", [t + 10], [0])]).clone())
        state = eng.cache.views[0].state.clone()
        return outs, state, eng

    with_graph, state_g, eng = run(True)
    without, state_n, _ = run(False)
    assert eng.graph_kernel_count(2) > 0
    assert sorted(state_g[:, 0].tolist()) == [4.0, 6.0] and torch.equal(state_g, state_n)
    for a, b in zip(with_graph, without):
        assert torch.allclose(a, b, rtol=0, atol=1e-5)


# ---------------------------------------------------------------------------------------------
# The decoder's optional constants: an architecture whose embedding rows are multiplied by a constant
# and whose logits are scaled and soft-capped is a parser only.

def register_toy_scaled():
    import dataclasses

    from blackwellllm_b200.config import register_architecture
    from blackwellllm_b200.models.dense_decoder import parse_dense_decoder

    def parse(raw):
        base = parse_dense_decoder(raw, architecture="ToyScaledForCausalLM", default_qkv_bias=False)
        return dataclasses.replace(base, embedding_multiplier=float(raw["embedding_multiplier"]),
                                   logit_scale=float(raw["logit_scale"]), logit_softcap=raw.get("final_logit_softcapping"))

    register_architecture("ToyScaledForCausalLM", parse)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("softcap", [None, 2.5])
def test_embedding_multiplier_logit_scale_and_soft_cap(dtype, softcap):
    from blackwellllm_b200 import Engine, StepEntry
    from blackwellllm_b200.weights.random_init import model_param_specs, random_tensors
    import tiny
    from plain_model import plain_config, plain_embedding, plain_layer
    register_toy_scaled()
    raw = dict(tiny.TINY_LLAMA, architectures=["ToyScaledForCausalLM"], embedding_multiplier=8.0, logit_scale=0.25)
    if softcap is not None:
        raw["final_logit_softcapping"] = softcap
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    W = random_tensors(model_param_specs(raw), seed=3, std=0.05, dtype=tdt)
    ids = tiny.prompt(37, raw["vocab_size"], 5)
    # the plain twin: the plain layers around the three constants
    c = plain_config(raw)
    Wd = {k: v.double() for k, v in W.items()}
    x = plain_embedding(Wd["model.embed_tokens.weight"], ids) * 8.0
    inv = plain_inv_freq(c["hd"], c["theta"], c["scaling"], c["rd"])
    for i in range(c["L"]):
        x = plain_layer(x, torch.arange(len(ids)), Wd, i, c, inv)
    ref = plain_linear(plain_rmsnorm(x, Wd["model.norm.weight"], c["eps"]), Wd["lm_head.weight"]) * 0.25
    if softcap is not None:
        ref = softcap * torch.tanh(ref / softcap)
    eng = Engine.from_tensors(raw, W, dtype=dtype, page_size=16, max_tokens=64, max_requests=1)
    out = torch.cat([eng.step([StepEntry("a", ids[:20], list(range(20)))]),
                     eng.step([StepEntry("a", ids[20:], list(range(17)))])]).double().cpu()
    tol = 1e-4 if dtype == "float32" else 1.5e-2
    assert float((out - ref).abs().max()) <= tol * float(ref.abs().max())
    plain_unscaled = plain_linear(plain_rmsnorm(x, Wd["model.norm.weight"], c["eps"]), Wd["lm_head.weight"])
    assert float((out - plain_unscaled).abs().max()) > 0.1 * float(plain_unscaled.abs().max())   # the constants matter
