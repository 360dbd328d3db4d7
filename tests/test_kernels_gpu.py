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
                                   (1000, 1111, 520), (2048, 1024, 4096)])
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
