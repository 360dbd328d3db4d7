"""Each CUDA kernel alone against a plain float32/float64 reference of the same op,
at sizes other than the tiny models': ragged, no power of two, edges of tiles."""
import math

import pytest
import torch

from plain_model import plain_attention, plain_inv_freq, plain_rmsnorm, plain_rope, plain_swiglu

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from blackwellllm_b200.kernels import ops as o
    return o


def rand(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


# ------------------------------------------------------------------ matrix products

@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (5, 300, 176), (8, 4096, 4096), (17, 136, 80), (64, 1000, 2048),
                                   (100, 6144, 1024), (256, 384, 96), (257, 512, 256), (300, 260, 200),
                                   (1000, 1111, 520), (2048, 1024, 4096),
                                   (2048, 4096, 64), (2048, 6144 + 48, 64),     # tiles 240 wide, the last one of a row cut
                                   (3, 19000, 200), (16, 25000, 136), (1, 128 * 149, 64 * 149),    # few tokens, more tiles than SMs: k-blocks dealt out in ranges
                                   (17, 19000, 200), (40, 25000, 136), (64, 128 * 149, 64 * 3)])   # the same up to 64 tokens
@pytest.mark.parametrize("mode", ["plain", "bias_f32out", "accumulate"])
def test_gemm_tc(ops, M, N, K, mode):
    x = rand(M, K, dtype=torch.bfloat16, seed=1).to(DEV)
    w = rand(N, K, dtype=torch.bfloat16, seed=2, scale=0.05).to(DEV)
    ref = x.double() @ w.double().T
    if mode == "plain":
        out = ops.gemm_tc(x, w)
        assert out.dtype == torch.bfloat16
        tol = 2 ** -8
    elif mode == "bias_f32out":
        b = rand(N, dtype=torch.bfloat16, seed=3).to(DEV)
        out = ops.gemm_tc(x, w, b, out_dtype=torch.float32)
        ref = ref + b.double()
        tol = 1e-5
    else:
        base = rand(M, N, seed=4).to(DEV)
        out = base.clone()
        ops.gemm_tc(x, w, out=out, accumulate=True)
        ref = ref + base.double()
        tol = 1e-5
    assert ops.gemm_tc_status() == 0
    scale = float(ref.abs().max())
    err = float((out.double() - ref).abs().max()) / scale
    assert err <= tol, f"{err:.3e}"


@pytest.mark.parametrize("splits", [2, 3, 8])
@pytest.mark.parametrize("M", [4, 200, 700])
def test_gemm_tc_split_k(ops, M, splits):
    N, K = 520, 2048 + 64 * 3
    x = rand(M, K, dtype=torch.bfloat16, seed=5).to(DEV)
    w = rand(N, K, dtype=torch.bfloat16, seed=6, scale=0.05).to(DEV)
    b = rand(N, seed=7).to(DEV)
    base = rand(M, N, seed=8).to(DEV)
    out = base.clone()
    ops.gemm_tc(x, w, b, out=out, accumulate=True, force_splits=splits)
    ref = x.double() @ w.double().T + b.double() + base.double()
    assert ops.gemm_tc_status() == 0
    assert float((out.double() - ref).abs().max()) / float(ref.abs().max()) <= 1e-5
    again = base.clone()
    ops.gemm_tc(x, w, b, out=again, accumulate=True, force_splits=splits)
    assert torch.equal(out, again)  # split sums are added in a fixed order


# ------------------------------------------------------------------ sums left to the reader

@pytest.mark.parametrize("M", [1, 3, 8, 16, 17, 64, 100, 256])
@pytest.mark.parametrize("N,K,force", [(4096, 4096, 0), (1000, 2056, 0), (6144, 512, 0), (384, 14336, 0), (520, 2240, 3),
                                       (128 * 149, 256, 0)])
def test_gemm_tc_planes_add_up_to_the_product(ops, M, N, K, force):
    x = rand(M, K, dtype=torch.bfloat16, seed=1).to(DEV)
    w = rand(N, K, dtype=torch.bfloat16, seed=2, scale=0.05).to(DEV)
    b = rand(N, seed=3).to(DEV)
    ref = x.double() @ w.double().T + b.double()
    planes = ops.gemm_tc_planes(x, w, b, force_splits=force)
    assert planes.dtype == torch.float32 and planes.shape[1:] == (M, N) and planes.shape[0] >= 1
    if force:
        assert planes.shape[0] == force
    if (N, K) == (384, 14336):
        assert planes.shape[0] > 1                  # three tiles and a long K: the planner splits
    if N == 128 * 149 and M <= 16:
        assert planes.shape[0] == 1                 # more tiles than SMs: one plane, written as the result
    total = planes[0].clone()
    for p in range(1, planes.shape[0]):
        total += planes[p]                          # the order in which the readers add them
    assert ops.gemm_tc_status() == 0
    assert float((total.double() - ref).abs().max()) / float(ref.abs().max()) <= 1e-5
    again = ops.gemm_tc_planes(x, w, b, force_splits=force).clone()
    assert torch.equal(again, ops.gemm_tc_planes(x, w, b, force_splits=force))
    with pytest.raises(ops.KernelError):
        ops.gemm_tc_planes(rand(257, K, dtype=torch.bfloat16).to(DEV), w)


@pytest.mark.parametrize("H,K", [(4096, 4096), (1000, 2056), (72, 200), (130, 14336)])
@pytest.mark.parametrize("odt", [torch.bfloat16, torch.float32])
def test_rmsnorm_adds_an_outstanding_sum(ops, H, K, odt):
    M, eps = 7, 1e-5
    x = rand(M, K, dtype=torch.bfloat16, seed=1).to(DEV)
    w = rand(H, K, dtype=torch.bfloat16, seed=2, scale=0.05).to(DEV)
    b = rand(H, seed=3).to(DEV)
    gain = (1 + rand(H, seed=4, scale=0.1)).to(odt).to(DEV)
    base = rand(M, H, seed=5).to(DEV)
    summed = base.double() + x.double() @ w.double().T + b.double()
    normed = summed * torch.rsqrt((summed * summed).mean(-1, keepdim=True) + eps) * gain.double()
    tol = 2 ** -8 if odt == torch.bfloat16 else 1e-5

    res = base.clone()
    ops.gemm_tc_deferred(x, w, b, res)
    assert ops.pending_target() is res and torch.equal(res, base)         # nothing was added yet
    out = ops.rmsnorm(res, gain, eps, odt)
    assert ops.pending_target() is None                                   # the norm added it and wrote the stream back
    assert float((res.double() - summed).abs().max()) / float(summed.abs().max()) <= 1e-5
    assert float((out.double() - normed).abs().max()) / float(normed.abs().max()) <= tol

    # chosen rows (they may repeat): the stream is left as it was and the sum stays outstanding
    res = base.clone()
    ops.gemm_tc_deferred(x, w, b, res)
    rows = torch.tensor([2, 0, 2, 6], dtype=torch.int32, device=DEV)
    out = ops.rmsnorm(res, gain, eps, odt, rows=rows)
    assert torch.equal(res, base) and ops.pending_target() is res
    assert float((out.double() - normed[rows.long()]).abs().max()) / float(normed.abs().max()) <= tol
    ops.resolve_pending()
    assert ops.pending_target() is None
    assert float((res.double() - summed).abs().max()) / float(summed.abs().max()) <= 1e-5

    # a norm that is refused (a gain of the wrong length) adds nothing: the sum stays outstanding
    res = base.clone()
    ops.gemm_tc_deferred(x, w, b, res)
    with pytest.raises(ops.KernelError):
        ops.rmsnorm(res, gain[:-1].contiguous(), eps, odt)
    assert ops.pending_target() is res and torch.equal(res, base)
    ops.resolve_pending()
    assert float((res.double() - summed).abs().max()) / float(summed.abs().max()) <= 1e-5


def test_an_outstanding_sum_is_made_before_anything_else_reads_or_replaces_it(ops):
    M, H, K = 5, 264, 520
    x = rand(M, K, dtype=torch.bfloat16, seed=1).to(DEV)
    w = rand(H, K, dtype=torch.bfloat16, seed=2, scale=0.05).to(DEV)
    base = rand(M, H, seed=5).to(DEV)
    summed = base.double() + x.double() @ w.double().T

    def close(t, ref):
        return float((t.double() - ref).abs().max()) / float(ref.abs().max()) <= 1e-5

    # another kernel of the package takes the tensor as an operand: the sum is made first
    res = base.clone()
    ops.gemm_tc_deferred(x, w, None, res)
    other = rand(M, H, seed=6).to(DEV)
    ops.rmsnorm(other, torch.ones(H, device=DEV), 1e-5, torch.float32)      # a norm of ANOTHER tensor leaves it alone
    assert ops.pending_target() is res
    ops.logit_transform(res, 2.0)
    assert ops.pending_target() is None and close(res, 2.0 * summed)

    # a second product is left open while the first still is: the first is added before its planes are overwritten
    res, res2 = base.clone(), base.clone()
    ops.gemm_tc_deferred(x, w, None, res)
    ops.gemm_tc_deferred(x, w, None, res2)
    assert ops.pending_target() is res2 and close(res, summed) and torch.equal(res2, base)
    ops.discard_pending(res)                      # not the outstanding one: nothing happens
    assert ops.pending_target() is res2
    ops.discard_pending(res2)
    assert ops.pending_target() is None and torch.equal(res2, base)


@pytest.mark.parametrize("nh,nkv,hd,rd,page", [(5, 1, 48, 32, 8), (4, 2, 64, 64, 16), (32, 8, 128, 128, 16)])
@pytest.mark.parametrize("M,force", [(3, 0), (16, 3), (8, 5)])
def test_rope_append_adds_planes(ops, nh, nkv, hd, rd, page, M, force):
    """The q/k/v product left as planes and rotated from there equals the rotation of the summed product, bit for bit
    where the sum is the same: compared with the same kernel on the planes added up beforehand in the same order."""
    K = 1024 + 64 * 5
    width = (nh + 2 * nkv) * hd
    x = rand(M, K, dtype=torch.bfloat16, seed=1).to(DEV)
    w = rand(width, K, dtype=torch.bfloat16, seed=2, scale=0.05).to(DEV)
    b = rand(width, seed=3).to(DEV)
    inv = (1e4 ** (-torch.arange(rd // 2, dtype=torch.float64) * 2 / rd)).float().to(DEV)
    positions = torch.arange(100, 100 + M, dtype=torch.int32, device=DEV)
    req = torch.zeros(M, dtype=torch.int32, device=DEV)
    n_pages = (100 + M) // page + 2
    table = torch.arange(n_pages, dtype=torch.int32, device=DEV).flip(0).reshape(1, -1).contiguous()
    pools = [torch.zeros(n_pages, nkv, page, hd, dtype=torch.bfloat16, device=DEV) for _ in range(4)]
    planes = ops.gemm_tc_planes(x, w, b, force_splits=force).clone()
    if force:
        assert planes.shape[0] == force
    total = planes[0].clone()
    for p in range(1, planes.shape[0]):
        total += planes[p]
    for paired in (False, True):
        q1 = ops.rope_append(planes, positions, req, table, inv, rd, pools[0], pools[1], nh, nkv, hd, paired=paired)
        q2 = ops.rope_append(total, positions, req, table, inv, rd, pools[2], pools[3], nh, nkv, hd, paired=paired)
        assert torch.equal(q1, q2) and torch.equal(pools[0], pools[2]) and torch.equal(pools[1], pools[3])
        assert float(pools[0].abs().max()) > 0


@pytest.mark.parametrize("mode", ["bias_accumulate", "swiglu", "bf16"])
@pytest.mark.parametrize("M,splits", [(300, 2), (700, 3), (1000, 4)])
def test_gemm_tc_split_k_on_cta_pairs(ops, M, splits, mode):
    """K splits of the CTA-pair kernel (steps of a few hundred tokens on products with few output features):
    every split writes its plane, the second kernel adds them in split order: right, and bit-equal when repeated."""
    N, K = 520, 2048 + 64 * 3
    x = rand(M, K, dtype=torch.bfloat16, seed=5).to(DEV)
    before = ops.gemm_pair_mode(2)       # pairs whenever they can
    try:
        if mode == "swiglu":
            I = 272
            wg = rand(I, K, dtype=torch.bfloat16, seed=2, scale=0.05).to(DEV)
            wu = rand(I, K, dtype=torch.bfloat16, seed=3, scale=0.05).to(DEV)
            w = ops.interleave_gate_up(wg, wu)
            run = lambda: ops.gemm_tc(x, w, swiglu=True, force_splits=splits)
            ref = plain_swiglu(x.double() @ wg.double().T, x.double() @ wu.double().T)
            tol = 2 ** -7
        else:
            w = rand(N, K, dtype=torch.bfloat16, seed=6, scale=0.05).to(DEV)
            if mode == "bf16":
                run = lambda: ops.gemm_tc(x, w, force_splits=splits)
                ref, tol = x.double() @ w.double().T, 2 ** -8
            else:
                b = rand(N, seed=7).to(DEV)
                base = rand(M, N, seed=8).to(DEV)

                def run():
                    out = base.clone()
                    ops.gemm_tc(x, w, b, out=out, accumulate=True, force_splits=splits)
                    return out
                ref, tol = x.double() @ w.double().T + b.double() + base.double(), 1e-5
        out = run()
        assert ops.gemm_tc_status() == 0
        assert float((out.double() - ref).abs().max()) <= tol * float(ref.abs().max())
        assert torch.equal(run(), out)
    finally:
        ops.gemm_pair_mode(before if before >= 0 else 1)


def test_gemm_tc_split_k_on_a_tile_width_that_is_no_power_of_two(ops):
    M, N, K = 2048, 4096, 256     # 16 x 18 tiles of 240 columns: the last one of a row is cut at 4096
    x = rand(M, K, dtype=torch.bfloat16, seed=5).to(DEV)
    w = rand(N, K, dtype=torch.bfloat16, seed=6, scale=0.05).to(DEV)
    out = ops.gemm_tc(x, w, out_dtype=torch.float32, force_splits=2)
    ref = x.double() @ w.double().T
    assert ops.gemm_tc_status() == 0
    assert float((out.double() - ref).abs().max()) / float(ref.abs().max()) <= 1e-5


@pytest.mark.parametrize("M,I,K,splits", [(1, 176, 64, 0), (8, 14336, 4096, 0), (33, 14336, 1024, 0), (64, 14336, 512, 0), (40, 1008, 512, 3), (300, 176, 256, 0),
                                          (700, 528, 2048, 2), (2048, 1024, 1024, 0),
                                          (2048, 14336, 64, 0)])   # tiles 224 wide
def test_gemm_tc_swiglu_epilogue(ops, M, I, K, splits):
    """silu(x Wg^T) * (x Wu^T) from the interleaved weight, in both orientations and with split-K."""
    x = rand(M, K, dtype=torch.bfloat16, seed=1).to(DEV)
    wg = rand(I, K, dtype=torch.bfloat16, seed=2, scale=0.05).to(DEV)
    wu = rand(I, K, dtype=torch.bfloat16, seed=3, scale=0.05).to(DEV)
    w = ops.interleave_gate_up(wg, wu)
    assert torch.equal(w[:16], wg[:16]) and torch.equal(w[16:32], wu[:16]) and torch.equal(w[32:48], wg[16:32])
    out = ops.gemm_tc(x, w, swiglu=True, force_splits=splits)
    assert out.shape == (M, I) and out.dtype == torch.bfloat16
    ref = plain_swiglu(x.double() @ wg.double().T, x.double() @ wu.double().T)
    assert ops.gemm_tc_status() == 0
    assert float((out.double() - ref).abs().max()) <= 2 ** -7 * float(ref.abs().max())


@pytest.mark.parametrize("M,splits", [(3, 0), (16, 3), (40, 2), (300, 0)])
@pytest.mark.parametrize("nh,nkv,hd,rd,page", [(5, 1, 48, 32, 8), (4, 2, 64, 64, 16), (2, 2, 16, 6, 4)])
def test_gemm_tc_rotary_epilogue(ops, M, splits, nh, nkv, hd, rd, page):
    """Projection + rotation + append in the product's epilogue, in every place it is written: sums
    inside the kernel (few tokens), the second kernel (more), the other orientation (many);
    head sizes where a warp of 32 features spans two heads, rotary sizes below the head size."""
    K = 264
    N = (nh + 2 * nkv) * hd
    w = rand(N, K, seed=1, scale=0.1).to(torch.bfloat16)
    b = rand(N, seed=2, scale=0.5).to(torch.bfloat16)
    x = rand(M, K, seed=3).to(torch.bfloat16)
    positions = torch.arange(M, dtype=torch.int32) * 3 + 1000          # far, and not consecutive
    n_blocks = (int(positions.max()) // page) + 1
    g = torch.Generator().manual_seed(4)
    num_pages = n_blocks + 5
    table = torch.randperm(num_pages, generator=g)[:n_blocks].to(torch.int32).view(1, n_blocks)
    req = torch.zeros(M, dtype=torch.int32)
    inv = plain_inv_freq(hd, 10000.0, None, rotary_dim=rd)
    order = ops.rotary_row_order(nh, nkv, hd, rd)
    kp = torch.zeros(num_pages, nkv, page, hd, dtype=torch.bfloat16, device=DEV)
    vp = torch.zeros_like(kp)
    tab = ops.rope_table(positions.to(DEV), inv.float().to(DEV), rd)
    slots = ops.kv_slots(positions.to(DEV), req.to(DEV), table.to(DEV), page, num_pages)
    q = ops.gemm_tc_rope(x.to(DEV), w[order].contiguous().to(DEV), b[order].contiguous().to(DEV), tab, slots, kp, vp,
                         nh, nkv, hd, rd, force_splits=splits)
    qkv = (x.double() @ w.double().T + b.double()).view(M, nh + 2 * nkv, hd)
    q_ref = plain_rope(qkv[:, :nh], positions, inv).reshape(M, nh * hd)
    k_ref = plain_rope(qkv[:, nh:nh + nkv], positions, inv)
    v_ref = qkv[:, nh + nkv:]
    tol = 2 ** -7
    assert float((q.double().cpu() - q_ref).abs().max()) <= tol * float(q_ref.abs().max())
    kc, vc = kp.double().cpu(), vp.double().cpu()
    for t in range(M):
        p_ = int(positions[t])
        pg = int(table[0, p_ // page])
        assert float((kc[pg, :, p_ % page] - k_ref[t]).abs().max()) <= tol * float(k_ref.abs().max())
        assert float((vc[pg, :, p_ % page] - v_ref[t]).abs().max()) <= tol * float(v_ref.abs().max())
    # nothing else in the pages was touched
    written = torch.zeros(num_pages, page, dtype=torch.bool)
    for t in range(M):
        p_ = int(positions[t])
        written[int(table[0, p_ // page]), p_ % page] = True
    assert float(kc.abs().amax(dim=(1, 3))[~written].max()) == 0.0
    # the same without an append: queries only
    kp.zero_()
    q2 = ops.gemm_tc_rope(x.to(DEV), w[order].contiguous().to(DEV), b[order].contiguous().to(DEV), tab, None, kp, vp,
                          nh, nkv, hd, rd, force_splits=splits)
    assert torch.equal(q2, q) and float(kp.abs().max()) == 0.0
    assert ops.gemm_tc_status() == 0


def test_gemm_tc_row_independent_of_batch(ops):
    """A token's row does not depend on which other tokens share the launch."""
    K, N = 1024, 768
    x = rand(64, K, dtype=torch.bfloat16, seed=9).to(DEV)
    w = rand(N, K, dtype=torch.bfloat16, seed=10, scale=0.05).to(DEV)
    whole = ops.gemm_tc(x, w, out_dtype=torch.float32)
    for rows in (slice(0, 1), slice(3, 20), slice(40, 64)):
        part = ops.gemm_tc(x[rows], w, out_dtype=torch.float32)
        assert float((part - whole[rows]).abs().max()) <= 1e-5 * float(whole.abs().max())


def test_gemm_tc_strided_input_and_refusals(ops):
    x_full = rand(10, 512, dtype=torch.bfloat16, seed=11).to(DEV)
    w = rand(72, 256, dtype=torch.bfloat16, seed=12).to(DEV)
    x = x_full[:, 256:]  # row stride 512, 16-byte aligned start
    out = ops.gemm_tc(x, w, out_dtype=torch.float32)
    ref = x.double() @ w.double().T
    assert float((out.double() - ref).abs().max()) <= 1e-5 * float(ref.abs().max())
    assert not ops.gemm_tc_supports(rand(4, 100, dtype=torch.bfloat16).to(DEV), rand(8, 100, dtype=torch.bfloat16).to(DEV))
    assert not ops.gemm_tc_supports(x_full[:, 1:257], w)  # start not 16-byte aligned
    with pytest.raises(ops.KernelError):
        ops.gemm_tc(rand(4, 100, dtype=torch.bfloat16).to(DEV), rand(8, 100, dtype=torch.bfloat16).to(DEV))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (3, 130, 100), (70, 65, 33), (129, 300, 176)])
def test_gemm_simt(ops, dtype, M, N, K):
    x = rand(M, K, dtype=dtype, seed=1).to(DEV)
    w = rand(N, K, dtype=dtype, seed=2).to(DEV)
    b = rand(N, seed=3).to(DEV)
    base = rand(M, N, seed=4).to(DEV)
    out = base.clone()
    ops.gemm_simt(x, w, b, out=out, accumulate=True)
    ref = x.double() @ w.double().T + b.double() + base.double()
    assert float((out.double() - ref).abs().max()) <= 2e-6 * float(ref.abs().max()) * math.sqrt(K)


# ------------------------------------------------------------------ row kernels

@pytest.mark.parametrize("H", [1, 48, 100, 1000, 4096, 5120 + 8])
@pytest.mark.parametrize("wdt,odt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                     (torch.float32, torch.bfloat16)])
def test_rmsnorm(ops, H, wdt, odt):
    x = rand(7, H, seed=1, scale=3.0).to(DEV)
    w = rand(H, dtype=wdt, seed=2).to(DEV)
    eps = 1e-5
    out = ops.rmsnorm(x, w, eps, odt)
    ref = plain_rmsnorm(x.double().cpu(), w.double().cpu(), eps)
    tol = 2e-6 if odt == torch.float32 else 2 ** -8
    assert float((out.double().cpu() - ref).abs().max()) <= tol * float(ref.abs().max())
    rows = torch.tensor([5, 0, 5, 2], dtype=torch.int32, device=DEV)
    sub = ops.rmsnorm(x, w, eps, odt, rows=rows)
    assert torch.equal(sub, out[rows.long()])


def test_rmsnorm_eps_matters(ops):
    x = torch.full((1, 64), 1e-3, device=DEV)
    w = torch.ones(64, device=DEV)
    a = ops.rmsnorm(x, w, 1e-5, torch.float32)
    b = ops.rmsnorm(x, w, 1e-6, torch.float32)
    assert abs(float(a[0, 0]) - 1e-3 / math.sqrt(1e-6 + 1e-5)) < 1e-6
    assert abs(float(b[0, 0]) - 1e-3 / math.sqrt(1e-6 + 1e-6)) < 1e-6


@pytest.mark.parametrize("table_dtype", [torch.float32, torch.bfloat16])
def test_embed_gather(ops, table_dtype):
    table = rand(301, 72, dtype=table_dtype, seed=1).to(DEV)
    ids = torch.tensor([300, 0, 7, 7, 150], dtype=torch.int32, device=DEV)
    out = ops.embed_gather(table, ids)
    assert out.dtype == torch.float32 and torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("I", [1, 176, 1000, 14336])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_swiglu(ops, I, dt):
    gu = rand(5, 2 * I, dtype=dt, seed=1, scale=2.0).to(DEV)
    out = ops.swiglu(gu)
    ref = plain_swiglu(gu[:, :I].double(), gu[:, I:].double())
    tol = 2e-6 if dt == torch.float32 else 2 ** -8
    assert float((out.double() - ref).abs().max()) <= tol * float(ref.abs().max())


# ------------------------------------------------------------------ attention over pages

class FakeBatch:
    """The fields of a step's batch that the attention kernels read."""

    def __init__(self, q_lens, kv_lens, static_bound=None):
        self.R = len(q_lens)
        self.h_q_len, self.h_kv_len = list(q_lens), list(kv_lens)
        self.h_q_start = [k - q for q, k in zip(q_lens, kv_lens)]
        cu = [0]
        for q in q_lens:
            cu.append(cu[-1] + q)
        self.T = cu[-1]
        i32 = dict(dtype=torch.int32, device=DEV)
        self.cu_q = torch.tensor(cu, **i32)
        self.q_start = torch.tensor(self.h_q_start, **i32)
        self.kv_len = torch.tensor(kv_lens, **i32)
        self.positions = torch.tensor([s + i for s, q in zip(self.h_q_start, q_lens) for i in range(q)], **i32)
        self.req_of_token = torch.tensor([r for r, q in enumerate(q_lens) for _ in range(q)], **i32)
        self.token_ids = self.positions
        self.static_bound = static_bound
        self.extras = {}
        self.static_extras = {}


def paged_case(q_lens, kv_lens, nh, nkv, hd, page, dtype, seed=0, spike=None):
    """Random q/k/v per request, keys and values scattered over shuffled pages (with
    unused pages full of NaN).  Returns what the kernels need and the plain result."""
    g = torch.Generator().manual_seed(seed)
    R = len(q_lens)
    blocks = [-(-k // page) for k in kv_lens]
    num_pages = sum(blocks) + 5
    perm = torch.randperm(num_pages, generator=g).tolist()
    k_pages = torch.full((num_pages, nkv, page, hd), float("nan"))
    v_pages = torch.full((num_pages, nkv, page, hd), float("nan"))
    width = max(blocks) + 2
    table = torch.full((R, width), -1, dtype=torch.int32)
    qs, refs = [], []
    for r in range(R):
        L, ql = kv_lens[r], q_lens[r]
        k = torch.randn(L, nkv, hd, generator=g).to(dtype).float()
        v = torch.randn(L, nkv, hd, generator=g).to(dtype).float()
        q = torch.randn(L, nh, hd, generator=g).to(dtype).float()
        if spike is not None:
            spike(r, q, k, v)
            q, k, v = q.to(dtype).float(), k.to(dtype).float(), v.to(dtype).float()
        ids = [perm.pop() for _ in range(blocks[r])]
        table[r, :blocks[r]] = torch.tensor(ids, dtype=torch.int32)
        for b, pid in enumerate(ids):
            n = min(page, L - b * page)
            k_pages[pid, :, :n] = k[b * page: b * page + n].transpose(0, 1)
            v_pages[pid, :, :n] = v[b * page: b * page + n].transpose(0, 1)
            # the rest of a request's last page keeps NaN: it must never be read into a result
        qs.append(q[L - ql:])
        refs.append((q, k, v, L - ql))
    return (torch.cat(qs).reshape(-1, nh * hd).to(dtype).to(DEV), k_pages.to(dtype).to(DEV),
            v_pages.to(dtype).to(DEV), table.to(DEV), refs)


def plain_rows(refs, window, nh, hd):
    outs = []
    for q, k, v, start in refs:
        o = plain_attention(q.double(), k.double(), v.double(), window=window)
        outs.append(o[start:].reshape(-1, nh * hd))
    return torch.cat(outs)


def run_attention(ops, dtype, q, kp, vp, table, batch, nh, window, scale):
    if dtype == torch.float32:
        return ops.attention_simt(q, kp, vp, batch.positions, batch.req_of_token, table, nh, window, scale)
    return ops.attention_mma(q, kp, vp, batch, table, nh, window, scale)


ATT_TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,page", [(4, 2, 16, 16), (3, 1, 32, 8), (8, 8, 64, 16), (32, 8, 128, 16),
                                            (14, 2, 48, 4), (6, 2, 256, 32), (5, 5, 80, 24)])
def test_attention_mixed_batch(ops, dtype, nh, nkv, hd, page):
    # prompt portions (one from position 0, one continuing), decode tokens, a two-token portion
    q_lens = [70, 1, 33, 2, 1, 130]
    kv_lens = [70, 200, 97, 64, 1, 400]
    q, kp, vp, table, refs = paged_case(q_lens, kv_lens, nh, nkv, hd, page, dtype, seed=hd)
    batch = FakeBatch(q_lens, kv_lens)
    out = run_attention(ops, dtype, q, kp, vp, table, batch, nh, None, hd ** -0.5)
    ref = plain_rows(refs, None, nh, hd)
    assert not torch.isnan(out).any()
    err = float((out.double().cpu() - ref).abs().max())
    assert err <= ATT_TOL[dtype] * float(ref.abs().max()), err


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [1, 7, 64, 100])
def test_attention_window(ops, dtype, window):
    nh, nkv, hd, page = 6, 2, 32, 8
    q_lens, kv_lens = [90, 1, 1, 3], [90, 300, 64, 131]
    q, kp, vp, table, refs = paged_case(q_lens, kv_lens, nh, nkv, hd, page, dtype, seed=window)
    # pages that every query's window has passed are gone from the block table
    for r, (ql, kl) in enumerate(zip(q_lens, kv_lens)):
        gone = max(0, (kl - ql) - window + 1) // page
        table[r, :gone] = -1
    batch = FakeBatch(q_lens, kv_lens)
    out = run_attention(ops, dtype, q, kp, vp, table, batch, nh, window, hd ** -0.5)
    ref = plain_rows(refs, window, nh, hd)
    assert not torch.isnan(out).any()
    assert float((out.double().cpu() - ref).abs().max()) <= ATT_TOL[dtype] * float(ref.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_far_key_and_window_edge(ops, dtype):
    """One key far back gets a score that dwarfs all others: the output must be its
    value.  With a window that ends one key after it, it must not be seen at all."""
    nh, nkv, hd, page = 4, 2, 64, 16
    L, far = 700, 3

    def spike(r, q, k, v):
        k[far] = 0
        k[far, :, 0] = 8.0
        q[-1] = 0
        q[-1, :, 0] = 8.0 * hd ** 0.5
        v[far] = 5.0

    for q_len in (1, 40):
        q, kp, vp, table, refs = paged_case([q_len], [L], nh, nkv, hd, page, dtype, seed=1, spike=spike)
        batch = FakeBatch([q_len], [L])
        out = run_attention(ops, dtype, q, kp, vp, table, batch, nh, None, hd ** -0.5)
        assert float((out[-1].float() - 5.0).abs().max()) < 0.05          # the far key wins
        w_in, w_out = L - far, L - far - 1                                 # window edge: in, then just out
        o_in = run_attention(ops, dtype, q, kp, vp, table, FakeBatch([q_len], [L]), nh, w_in, hd ** -0.5)
        o_out = run_attention(ops, dtype, q, kp, vp, table, FakeBatch([q_len], [L]), nh, w_out, hd ** -0.5)
        assert float((o_in[-1].float() - 5.0).abs().max()) < 0.05
        assert float(o_out[-1].float().abs().max()) < 4.0
        ref = plain_rows(refs, w_out, nh, hd)
        assert float((o_out.double().cpu() - ref).abs().max()) <= ATT_TOL[dtype] * float(ref.abs().max())


@pytest.mark.parametrize("nh,nkv,hd,rd,page", [(8, 2, 128, 128, 16), (4, 4, 64, 64, 8), (16, 1, 192, 64, 32), (6, 2, 128, 0, 64)])
@pytest.mark.parametrize("window,append", [(None, True), (100, True), (None, False)])
def test_decode_attention_rotates_and_appends_from_the_unsummed_product(ops, nh, nkv, hd, rd, page, window, append):
    """One token per request: the key-slice kernel makes the rotated queries, and the token's rotated key and its
    value, from the planes of the q/k/v product itself and writes key and value to the cache.  Compared with the
    rotation kernel followed by the same attention on a cache of its own: the same output and the same pages
    (up to the last bit of a bfloat16: the two kernels' products may be contracted differently).  The tokens'
    positions sit in the middle of a tile, at a tile's and a page's first and last key, and alone in a cache."""
    kv_lens = [1, 17, 64, 65, 200, 1000, 3000, 128, 4 * page + 1]
    R = len(kv_lens)
    q_lens = [1] * R
    K = 1024 + 64 * 3
    width = (nh + 2 * nkv) * hd
    x = rand(R, K, dtype=torch.bfloat16, seed=1).to(DEV)
    w = rand(width, K, dtype=torch.bfloat16, seed=2, scale=0.05).to(DEV)
    b = rand(width, seed=3, scale=0.3).to(DEV)
    _, kp, vp, table, _ = paged_case(q_lens, kv_lens, nh, nkv, hd, page, torch.bfloat16, seed=7)
    # the cache's rows of the tokens' own positions hold what an earlier user of the page left: NaN
    batch = FakeBatch(q_lens, kv_lens)
    for r, L in enumerate(kv_lens):
        pid, slot = int(table[r, (L - 1) // page]), (L - 1) % page
        if append:
            kp[pid, :, slot] = float("nan"); vp[pid, :, slot] = float("nan")
    inv = (1e4 ** (-torch.arange(rd // 2, dtype=torch.float64) * 2 / max(rd, 1))).float().to(DEV)
    tab = ops.rope_table(batch.positions, inv, rd) if rd else None
    planes = ops.gemm_tc_planes(x, w, b, force_splits=3).clone()
    caches = [(kp.clone(), vp.clone()) for _ in range(2)]
    q = ops.rope_append(planes, batch.positions, batch.req_of_token, table, inv if rd else None, rd, caches[0][0], caches[0][1],
                        nh, nkv, hd, append=append, table=tab, paired=True)
    ref = ops.attention_mma(q, caches[0][0], caches[0][1], batch, table, nh, window, hd ** -0.5)
    raw = ops.UnrotatedQKV(planes, tab, rd, append, None)
    out = ops.attention_mma(raw, caches[1][0], caches[1][1], FakeBatch(q_lens, kv_lens), table, nh, window, hd ** -0.5)
    assert not torch.isnan(out).any() and not torch.isnan(ref).any()
    assert float((out.float() - ref.float()).abs().max()) <= ATT_TOL[torch.bfloat16] * float(ref.float().abs().max())
    for mine, theirs in zip(caches[1], caches[0]):
        same_nan = torch.isnan(mine) == torch.isnan(theirs)
        assert bool(same_nan.all())                                    # exactly the same rows were written
        a, c = torch.nan_to_num(mine.float()), torch.nan_to_num(theirs.float())
        assert float((a - c).abs().max()) <= 2 ** -7 * float(c.abs().max())
    if append:
        for r, L in enumerate(kv_lens):                                # and they were written: no NaN is left there
            pid, slot = int(table[r, (L - 1) // page]), (L - 1) % page
            assert not torch.isnan(caches[1][0][pid, :, slot]).any() and not torch.isnan(caches[1][1][pid, :, slot]).any()
    with pytest.raises(ops.KernelError):                               # a request with two tokens: refused
        ops.attention_mma(raw, caches[1][0], caches[1][1], FakeBatch([1] * (R - 1) + [2], kv_lens), table, nh, window, hd ** -0.5)
    live = ops.UnrotatedQKV(ops.gemm_tc_planes(x, w, b), tab, rd, append, None)
    ops.gemm_tc_planes(x, w, b)                                        # a later product takes the plane buffer
    with pytest.raises(ops.KernelError, match="overwritten"):
        ops.attention_mma(live, caches[1][0], caches[1][1], FakeBatch(q_lens, kv_lens), table, nh, window, hd ** -0.5)


def test_attention_decode_slices_and_static_bound(ops):
    """Long decode rows are cut into key slices; a graph-style static bound changes
    the number of slices but not the result beyond rounding."""
    nh, nkv, hd, page = 8, 2, 128, 16
    q_lens, kv_lens = [1, 1, 2], [3000, 17, 1025]
    q, kp, vp, table, refs = paged_case(q_lens, kv_lens, nh, nkv, hd, page, torch.bfloat16, seed=5)
    ref = plain_rows(refs, None, nh, hd)
    a = ops.attention_mma(q, kp, vp, FakeBatch(q_lens, kv_lens), table, nh, None, hd ** -0.5)
    b = ops.attention_mma(q, kp, vp, FakeBatch(q_lens, kv_lens, static_bound=8192), table, nh, None, hd ** -0.5)
    for out in (a, b):
        assert float((out.double().cpu() - ref).abs().max()) <= 2e-2 * float(ref.abs().max())
    assert float((a.float() - b.float()).abs().max()) <= 2e-2 * float(ref.abs().max())
