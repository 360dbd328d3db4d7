"""The tensor-core product's planner (``bw_gemm_tc_plan`` in csrc/gemm_tc.cu) is host code:
which orientation, which tile width and how many K splits a product gets.  Its
decisions are checked here without a GPU, over the shapes the engine's layers produce and
over odd ones: every decision must be one the kernels are built for, and a split must fit
the scratch it is given."""
import ctypes
import itertools

import pytest

BM, BK, NUM_SMS = 128, 64, 148          # csrc/gemm_tc.cu: tile rows, k-block, CTAs of the persistent grid
WIDTHS_TOKENS_WIDE = (16, 32, 64, 128, 256)   # features in the 128-row dimension: tokens rounded up to a power of two
WIDTHS_FEATURES_WIDE = (128, 224, 240, 256)   # tokens in the 128-row dimension


@pytest.fixture(scope="module")
def plan():
    from blackwellllm_b200.kernels.build import load_library
    lib = load_library("gemm_tc")
    fn = lib.bw_gemm_tc_plan
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_longlong, ctypes.c_longlong,
                   ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]

    def call(M, N, K, swiglu=0, workspace=1 << 24, counters=1 << 14):
        tr, bn = ctypes.c_int(-1), ctypes.c_int(-1)
        splits = fn(M, N, K, swiglu, workspace, counters, ctypes.byref(tr), ctypes.byref(bn))
        return splits, tr.value, bn.value
    return call


def ceil_div(a, b):
    return -(-a // b)


TOKENS = (1, 2, 3, 7, 8, 16, 17, 33, 64, 65, 100, 128, 255, 256, 257, 300, 512, 1000, 1024, 2048, 2049, 8192)
# (features, inner size): q/k/v, o, gate/up, down and head of the three layer shapes the bench knows, and odd ones
PRODUCTS = ((6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336), (128256, 4096),
            (4608, 3584), (3584, 3584), (37888, 3584), (3584, 18944), (152064, 3584),
            (7168, 5120), (5120, 5120), (27648, 5120), (5120, 13824),
            (16, 8), (48, 24), (100, 72), (352, 64), (1000, 1000), (33, 4096))


@pytest.mark.parametrize("swiglu", (0, 1))
def test_every_decision_is_one_the_kernels_are_built_for(plan, swiglu):
    for M, (N, K) in itertools.product(TOKENS, PRODUCTS):
        if swiglu and N % 32:
            continue
        splits, tr, bn = plan(M, N, K, swiglu)
        what = f"M={M} N={N} K={K} swiglu={swiglu}: splits={splits} transposed={tr} bn={bn}"
        assert tr == (1 if M <= 256 else 0), what
        if tr:
            assert bn in WIDTHS_TOKENS_WIDE and bn >= M and (bn == 16 or bn // 2 < M), what
        else:
            assert bn in WIDTHS_FEATURES_WIDE, what
            assert not swiglu or bn % 32 == 0, what      # the SwiGLU epilogue pairs 16 gate with 16 up features
        kb_total = ceil_div(K, BK)
        assert 1 <= splits <= max(1, kb_total), what
        tiles = ceil_div(N, BM) * ceil_div(M, bn) if tr else ceil_div(M, BM) * ceil_div(N, bn)
        if tiles >= NUM_SMS:
            assert splits == 1, what                        # enough tiles for every CTA: no partial sums
        if splits > 1:
            assert splits <= 16 and kb_total // splits >= 8, what
            assert M <= 64 or splits * 8 * M <= K, what     # partial sums stay well below the weight bytes


def test_a_split_fits_the_scratch_it_is_given(plan):
    for M, (N, K) in itertools.product((1, 8, 16, 64, 200), PRODUCTS):
        free, tr, bn = plan(M, N, K)
        tiles = ceil_div(N, BM) * ceil_div(M, bn)
        for workspace, counters in ((0, 0), (M * N, 1 << 14), (3 * M * N, 1 << 14), (1 << 24, 4 * tiles - 1),
                                    (1 << 24, 4 * tiles)):
            splits, tr2, bn2 = plan(M, N, K, 0, workspace, counters)
            assert (tr2, bn2) == (tr, bn)                   # scratch changes the split only
            assert 1 <= splits <= free
            if splits > 1:
                assert splits * M * N <= workspace and tiles * 4 <= counters


def test_decode_shapes_fill_the_gpu(plan):
    """The products of a decode step at batch 1 to 64 on the 8B layer sizes: with fewer tiles than
    CTAs the K splits bring the items of a round to at least half of the CTAs."""
    for M in (1, 8, 64):
        for N, K in ((6144, 4096), (4096, 4096), (4096, 14336)):
            splits, tr, bn = plan(M, N, K)
            tiles = ceil_div(N, BM) * ceil_div(M, bn)
            assert tr == 1 and tiles < NUM_SMS
            assert NUM_SMS // 2 <= tiles * splits <= NUM_SMS, (M, N, K, splits)


def test_pair_plan_splits_k_only_where_the_pairs_would_idle():
    """CTA pairs for more than 256 tokens: K is split only where it was measured to pay: in two halves, a long K
    (the down projection) at a few hundred tokens, when both halves of every tile fit one round of the 74 pairs."""
    from blackwellllm_b200.kernels.build import load_library
    lib = load_library("gemm_tc")
    fn = lib.bw_gemm_tc_pair_plan
    fn.restype = ctypes.c_double
    fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_longlong,
                   ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]

    def plan(M, N, K, force=0, workspace=1 << 24):
        wd, sp = ctypes.c_int(-1), ctypes.c_int(-1)
        cost = fn(M, N, K, force, workspace, ctypes.byref(wd), ctypes.byref(sp))
        return cost, wd.value, sp.value

    for M in (300, 512, 1024, 2048, 8192):
        for N, K in PRODUCTS[:14]:
            cost, wd, sp = plan(M, N, K)
            assert cost > 0 and wd in (224, 256) and 1 <= sp <= 4, (M, N, K)
            kb = ceil_div(K, BK)
            tiles = ceil_div(M, 2 * BM) * ceil_div(N, wd)
            if sp > 1:   # two halves of a long K whose items fit one round of the 74 pairs, planes within the scratch
                assert sp == 2 and kb >= 128 and tiles * 2 <= NUM_SMS // 2 and sp * M * N <= 1 << 24
            assert plan(M, N, K, workspace=0)[2] == 1            # no scratch, no split
    assert plan(512, 4096, 14336)[2] == 2                        # down at 512 tokens: 32 tiles for 74 pairs
    assert plan(512, 4096, 4096)[2] == 1 and plan(768, 4096, 14336)[2] == 1
    assert plan(2048, 28672, 4096)[2] == 1                       # gate/up at 2,048 tokens: rounds of whole tiles
    assert plan(700, 520, 2240, force=3)[2] == 3                 # a forced split is taken as it is
