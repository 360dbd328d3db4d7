"""The allocation-free entry point of the tensor-core matrix product, called through
its exported C symbol, against the regular entry point.

Some users of the library cannot allocate device memory when they call it (inside a
stream capture, under a fixed memory budget, in a loop whose owner forbids every
allocating call).  ``bw_gemm_tc_noalloc`` keeps its split-K partial sums in a static
device array of 4 Mi floats that the library brings along; the regular entry point
is handed a workspace by the caller.  Both must give the same numbers.

Collected last on purpose (file name), so that a run that stops at the first
failure has already run every other test.  It stands alone as well: it builds and
loads its own library and shares no state with the other tests.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCRATCH_FLOATS = 4 * 1024 * 1024
TOO_LARGE = -10


def _entry():
    from blackwellllm_b200.kernels.build import load_library
    lib = load_library("gemm_tc_noalloc")
    fn = lib.bw_gemm_tc_noalloc
    vp, i, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    fn.argtypes = [vp, vp, vp, i, vp, i, i, i, i, ll, ll, i, i, vp]
    fn.restype = i
    lib.bw_gemm_tc_status.argtypes = []
    lib.bw_gemm_tc_status.restype = i
    return fn, lib.bw_gemm_tc_status


def _call(fn, x, w, bias, out, accumulate, splits):
    M, K = x.shape
    N = w.shape[0]
    code = {torch.float32: 0, torch.bfloat16: 1}
    return fn(x.data_ptr(), w.data_ptr(), 0 if bias is None else bias.data_ptr(),
              0 if bias is None else code[bias.dtype], out.data_ptr(), code[out.dtype], M, N, K,
              x.stride(0), out.stride(0), int(accumulate), splits,
              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def _case(M, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    bias = torch.randn(N, generator=g).to(DEV)
    base = torch.randn(M, N, generator=g).to(DEV)
    return x, w, bias, base


def test_no_alloc_entry_matches_the_regular_one_twice_in_a_row():
    from blackwellllm_b200.kernels import ops
    fn, status = _entry()
    # the second call is smaller, so the scratch still holds the first call's sums around its own
    for (M, N, K, splits, seed) in [(48, 1000, 2048, 4, 1), (5, 520, 1024 + 192, 3, 2)]:
        x, w, bias, base = _case(M, N, K, seed)
        mine = base.clone()
        assert _call(fn, x, w, bias, mine, True, splits) == 0     # the first call also loads the kernels
        torch.cuda.synchronize()
        mine.copy_(base)
        # what the DEVICE reports as free (cudaMemGetInfo: it sees every allocation, whoever makes it) and
        # torch's own counter, around a call that is complete before the second reading
        free_before, held_before = torch.cuda.mem_get_info(DEV)[0], torch.cuda.memory_allocated(DEV)
        rc = _call(fn, x, w, bias, mine, True, splits)
        torch.cuda.synchronize()
        assert rc == 0, rc
        assert torch.cuda.mem_get_info(DEV)[0] == free_before and torch.cuda.memory_allocated(DEV) == held_before
        assert status() == 0                                      # this library's own bounded waits never gave up
        theirs = base.clone()
        ops.gemm_tc(x, w, bias, out=theirs, accumulate=True, force_splits=splits)
        torch.cuda.synchronize()
        ref = x.double() @ w.double().T + bias.double() + base.double()
        scale = float(ref.abs().max())
        assert float((mine.double() - ref).abs().max()) <= 1e-5 * scale
        assert float((mine - theirs).abs().max()) <= 1e-5 * scale
        # bfloat16 output, no accumulate, same scratch again
        out16 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        assert _call(fn, x, w, None, out16, False, splits) == 0
        ref16 = x.double() @ w.double().T
        assert float((out16.double() - ref16).abs().max()) <= 2 ** -8 * float(ref16.abs().max())


def test_no_alloc_entry_refuses_what_its_scratch_cannot_hold():
    fn, status = _entry()
    M, N, K = 256, 8192, 1024           # 4 splits x 256 x 8192 floats > 4 Mi
    x, w, _, _ = _case(M, N, K, 3)
    out = torch.full((M, N), 7.0, device=DEV)
    assert 4 * M * N > SCRATCH_FLOATS
    assert _call(fn, x, w, None, out, False, 4) == TOO_LARGE
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())      # nothing was launched
    assert _call(fn, x, w, None, out, False, 2) == 0   # 2 x 256 x 8192 = 4 Mi floats: just fits
    ref = x.double() @ w.double().T
    assert float((out.double() - ref).abs().max()) <= 1e-5 * float(ref.abs().max())
    # one split uses neither array: a product far beyond the scratch goes through
    M, N, K = 2048, 4096, 512
    x, w, _, _ = _case(M, N, K, 4)
    big = torch.empty(M, N, device=DEV)
    assert M * N > SCRATCH_FLOATS and _call(fn, x, w, None, big, False, 1) == 0
    ref = x.double() @ w.double().T
    assert float((big.double() - ref).abs().max()) <= 1e-5 * float(ref.abs().max())
    # more output tiles than there are counters: the documented code, nothing launched
    M, N, K = 1, 128 * 4100, 128
    x, w, _, _ = _case(M, N, K, 5)
    row = torch.full((M, N), 7.0, device=DEV)
    assert 2 * M * N <= SCRATCH_FLOATS and _call(fn, x, w, None, row, False, 2) == TOO_LARGE
    torch.cuda.synchronize()
    assert bool((row == 7.0).all()) and status() == 0
