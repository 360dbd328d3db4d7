// bfloat16 matrix product on the 5th-generation tensor cores:
//     acc[i, j] = sum_k A[i, k] * B[j, k]      (A: [Ra, K], B: [Rb, K], both row-major)
// TMA brings 128 x 64 tiles of A and BN x 64 tiles of B into shared memory (128-byte
// swizzle), one elected thread issues tcgen05.mma into a TMEM accumulator, and four
// epilogue warps read it back with tcgen05.ld.  Each CTA loads its own tiles (no
// multicast).  One output tile per CTA; split-K over gridDim.z writes float32
// partials that a second kernel sums in split order (deterministic).
//
// The same kernel serves both orientations of  out[tokens, features] = x . w^T:
//   normal     A = x (tokens),   B = w (features): prefill, many tokens;
//   transposed A = w (features), B = x (tokens):   few tokens (decode): the weight
//              rows fill the 128-row MMA dimension and the tokens are the narrow N.
// Epilogue: + bias[feature], then store (float32 | bfloat16) or add into float32 out.
//
// Roles (192 threads): warp 0 TMA producer, warp 1 TMEM owner + MMA issuer,
// warps 2..5 epilogue (TMEM lane quarter = warp % 4).  Every wait is bounded; a
// timeout sets the status word, and all roles fall through to the common exit
// where TMEM is freed.
#include "tcgen05.cuh"

using bf16 = __nv_bfloat16;

namespace {

constexpr int BM = 128;       // rows of the A tile = MMA M
constexpr int BK = 64;        // k-block: 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;
constexpr int THREADS = 192;
constexpr int SMEM_BUDGET = 200 * 1024;

__device__ int g_status = 0;  // 0 ok; else the code of the first wait that gave up

struct Epilogue {
    void* out;            // [tokens, features], row stride ldo (elements)
    float* partial;       // split-K: [splits, tokens, features] dense float32; else null
    const void* bias;     // [features] or null
    long long ldo;
    int out_type, bias_type, accumulate, transposed;
    int tokens, features;
};

// Wide tiles take the whole SM; narrow ones (few tokens: a weight stream bound by HBM) use 4
// stages so that 2-3 CTAs share an SM and one CTA's start-up and epilogue overlap the others' loads.
template <int BN> __host__ __device__ constexpr int stages_for() {
    constexpr int per = A_BYTES + BN * BK * 2;
    constexpr int s = SMEM_BUDGET / per;
    return BN <= 64 ? 4 : (s > 8 ? 8 : s);
}
constexpr int ctas_per_sm(int bn) { return bn <= 16 ? 3 : (bn <= 64 ? 2 : 1); }

__device__ __forceinline__ void store_val(const Epilogue& ep, int token, int feature, float v) {
    if (ep.bias) v += ep.bias_type == BW_F32 ? ((const float*)ep.bias)[feature]
                                              : __bfloat162float(((const bf16*)ep.bias)[feature]);
    const size_t off = (size_t)token * ep.ldo + feature;
    if (ep.out_type == BW_F32) {
        float* o = (float*)ep.out + off;
        *o = ep.accumulate ? *o + v : v;
    } else {
        ((bf16*)ep.out)[off] = __float2bfloat16_rn(v);
    }
}

template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               Epilogue ep, int kb_total, int kb_per_split) {
    constexpr int STAGES = stages_for<BN>();
    constexpr int B_BYTES = BN * BK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
    constexpr uint32_t IDESC = bw::umma_idesc_bf16(BM, BN);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES);   // full[STAGES], empty[STAGES], tmem_full
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_a = blockIdx.x, tile_b = blockIdx.y, split = blockIdx.z;
    const int kb0 = split * kb_per_split;
    const int nkb = min(kb_total, kb0 + kb_per_split) - kb0;

    const uint32_t full0 = bw::smem_u32(bars), empty0 = bw::smem_u32(bars + STAGES);
    const uint32_t tmem_full = bw::smem_u32(bars + 2 * STAGES);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { bw::mbar_init(full0 + 8 * s, 1); bw::mbar_init(empty0 + 8 * s, 1); }
        bw::mbar_init(tmem_full, 1);
        bw::fence_barrier_init();
        bw::tma_prefetch_desc(&tmA);
        bw::tma_prefetch_desc(&tmB);
        tmem_slot[1] = (uint32_t)g_status;   // an earlier timeout: later CTAs do no work
    }
    if (warp == 1) bw::tmem_alloc(bw::smem_u32(tmem_slot), TMEM_COLS);
    bw::tc_fence_before();
    __syncthreads();
    bw::tc_fence_after();
    const uint32_t tmem_acc = *tmem_slot;
    const bool dead = tmem_slot[1] != 0;

    if (dead) {
        // fall through to the exit
    } else if (warp == 0) {
        if (lane == 0) {
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                const uint32_t ph = (i / STAGES) & 1;
                if (!bw::mbar_wait(empty0 + 8 * s, ph ^ 1, &g_status, 1)) break;
                bw::mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                const uint32_t a_dst = bw::smem_u32(smem + s * STAGE_BYTES);
                bw::tma_load_2d(a_dst, &tmA, full0 + 8 * s, (kb0 + i) * BK, tile_a * BM);
                bw::tma_load_2d(a_dst + A_BYTES, &tmB, full0 + 8 * s, (kb0 + i) * BK, tile_b * BN);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            for (int i = 0; i < nkb && ok; ++i) {
                const int s = i % STAGES;
                const uint32_t ph = (i / STAGES) & 1;
                ok = bw::mbar_wait(full0 + 8 * s, ph, &g_status, 2);
                if (!ok) break;
                bw::tc_fence_after();
                const uint32_t a_addr = bw::smem_u32(smem + s * STAGE_BYTES);
                const uint64_t da = bw::umma_smem_desc_sw128(a_addr);
                const uint64_t db = bw::umma_smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    // advance 32 bytes (2 units of 16 B) along K inside the swizzle row
                    bw::umma_bf16(tmem_acc, da + 2 * k, db + 2 * k, IDESC, (i | k) != 0);
                }
                bw::umma_commit(empty0 + 8 * s);   // the stage is free once these MMAs are done
            }
            bw::umma_commit(tmem_full);            // the accumulator is complete
        }
    } else {
        const int quarter = warp & 3;              // TMEM lanes 32 * quarter .. + 31
        const int row = quarter * 32 + lane;       // row of the A tile
        const int ga = tile_a * BM + row;          // global A row
        if (bw::mbar_wait(tmem_full, 0, &g_status, 3)) {
            bw::tc_fence_after();
            const uint32_t lane_addr = tmem_acc + ((uint32_t)(quarter * 32) << 16);
            const int a_rows = ep.transposed ? ep.features : ep.tokens;
            const int b_rows = ep.transposed ? ep.tokens : ep.features;
            float* part = ep.partial ? ep.partial + (size_t)split * ep.tokens * ep.features : nullptr;
            constexpr int CH = BN < 32 ? 16 : 32;
            // All MMAs are complete, so the pipeline's shared memory is free: each epilogue
            // warp takes 32 x 33 floats of it to turn its 32 x 32 block, so that in the
            // normal orientation a warp stores whole rows (32 consecutive features).
            float* stage = (float*)smem + (warp - 2) * (32 * 33);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += CH) {
                uint32_t v[CH];
                if constexpr (CH == 32) bw::tmem_ld_32x32(lane_addr + c0, v);
                else bw::tmem_ld_32x16(lane_addr + c0, v);
                bw::tmem_ld_wait();
                if (ep.transposed) {
                    // lanes hold consecutive features of one token per column: already coalesced
                    if (ga < a_rows) {
#pragma unroll
                        for (int c = 0; c < CH; ++c) {
                            const int token = tile_b * BN + c0 + c;
                            if (token < b_rows) {
                                const float acc = __uint_as_float(v[c]);
                                if (part) part[(size_t)token * ep.features + ga] = acc;
                                else store_val(ep, token, ga, acc);
                            }
                        }
                    }
                } else {
                    if constexpr (CH == 32) {
#pragma unroll
                        for (int c = 0; c < 32; ++c) stage[lane * 33 + c] = __uint_as_float(v[c]);
                        __syncwarp();
                        const int feature = tile_b * BN + c0 + lane;
                        if (feature < b_rows) {
#pragma unroll 4
                            for (int r = 0; r < 32; ++r) {
                                const int token = tile_a * BM + quarter * 32 + r;
                                if (token >= a_rows) break;
                                const float acc = stage[r * 33 + lane];
                                if (part) part[(size_t)token * ep.features + feature] = acc;
                                else store_val(ep, token, feature, acc);
                            }
                        }
                        __syncwarp();
                    }
                }
            }
        }
    }
    bw::tc_fence_before();
    __syncthreads();
    if (warp == 1) bw::tmem_dealloc(tmem_acc, TMEM_COLS);
}

// out = (accumulate ? out : 0) + bias + sum over splits of partial, in split order
__global__ void splitk_reduce_kernel(Epilogue ep, int splits) {
    const size_t total = (size_t)ep.tokens * ep.features;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < splits; ++s) v += ep.partial[(size_t)s * total + i];
        const int token = (int)(i / ep.features), feature = (int)(i - (size_t)token * ep.features);
        store_val(ep, token, feature, v);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = (EncodeTiledFn)p;
    }
    return fn;
}

// rows x K bf16 matrix with row stride ld (elements), box = box_rows x 64, 128-byte swizzle
bool make_map(CUtensorMap* m, const void* base, long long rows, long long K, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN>
int launch(const CUtensorMap& a, const CUtensorMap& b, const Epilogue& ep, dim3 grid, int kb_total,
           int kb_per_split, cudaStream_t s) {
    constexpr int STAGES = stages_for<BN>();
    constexpr int smem = STAGES * (A_BYTES + BN * BK * 2) + (2 * STAGES + 1) * 8 + 16 + 1024;
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    gemm_tc_kernel<BN><<<grid, THREADS, smem, s>>>(a, b, ep, kb_total, kb_per_split);
    BW_LAUNCH_CHECK();
    return 0;
}

int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

}  // namespace

// Whether bw_gemm_tc takes these operands: bf16, K a multiple of 8 (a TMA row stride
// is a multiple of 16 bytes), 16-byte aligned bases and strides.
BW_EXPORT int bw_gemm_tc_supported(const void* x, const void* w, int K, long long ldx) {
    return (K > 0 && K % 8 == 0 && ldx % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0) ? 1 : 0;
}

// Picks the orientation, the tile width and the number of K splits for
// out[M, N] = x[M, K] . w[N, K]^T.  Returns splits; *transposed and *bn are set.
BW_EXPORT int bw_gemm_tc_plan(int M, int N, int K, long long workspace_elems, int* transposed, int* bn) {
    const int kb_total = ceil_div(K, BK);
    int tr = M <= 256, b;
    if (tr) { b = 16; while (b < M) b *= 2; }
    else {
        // wave efficiency on 148 SMs picks between 128- and 256-wide tiles
        auto eff = [&](int w) { long long t = (long long)ceil_div(M, BM) * ceil_div(N, w);
                                return (double)t / ((double)ceil_div(t, 148) * 148) * (w == 256 ? 1.0 : 0.92); };
        b = eff(256) >= eff(128) ? 256 : 128;
    }
    *transposed = tr; *bn = b;
    const long long tiles = tr ? (long long)ceil_div(N, BM) * ceil_div(M, b) : (long long)ceil_div(M, BM) * ceil_div(N, b);
    int best = 1; double best_score = 0;
    for (int s = 1; s <= 8; ++s) {
        if (s > 1 && (kb_total / s < 8 || (long long)s * M * N > workspace_elems)) break;
        const long long ctas = tiles * s, slots = 148LL * ctas_per_sm(b);
        const double wave = (double)ctas / ((double)ceil_div(ctas, slots) * slots);
        const double extra = s > 1 ? 4.0 * s * M / (double)K : 0.0;   // partial traffic relative to the weights
        const double score = wave / (1.0 + extra);
        if (score > best_score * 1.02) { best_score = score; best = s; }
    }
    return best;
}

// out[M, N] (=|+=) x[M, K] . w[N, K]^T (+ bias[N]).  x, w bf16; out float32 or bf16
// (accumulate: float32).  workspace: float32 scratch for split-K partials (may be null).
// force_splits > 0 overrides the planner (tests).
BW_EXPORT int bw_gemm_tc(const void* x, const void* w, const void* bias, int bias_type, void* out, int out_type,
                         int M, int N, int K, long long ldx, long long ldo, int accumulate, float* workspace,
                         long long workspace_elems, int force_splits, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (!bw_gemm_tc_supported(x, w, K, ldx)) return BW_ERR_UNSUPPORTED;
    if (accumulate && out_type != BW_F32) return BW_ERR_BAD_ARG;
    if (ldo < N) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    int tr, bn;
    int splits = bw_gemm_tc_plan(M, N, K, workspace ? workspace_elems : 0, &tr, &bn);
    const int kb_total = ceil_div(K, BK);
    if (force_splits > 0) {
        splits = force_splits;
        if (splits > kb_total) splits = kb_total;
        if (splits > 1 && (!workspace || (long long)splits * M * N > workspace_elems)) return BW_ERR_BAD_ARG;
    }
    int kb_per_split = ceil_div(kb_total, splits);
    splits = ceil_div(kb_total, kb_per_split);   // no empty split

    CUtensorMap ta, tb;
    const void* a_ptr = tr ? w : x; const void* b_ptr = tr ? x : w;
    const long long a_rows = tr ? N : M, b_rows = tr ? M : N;
    const long long a_ld = tr ? K : ldx, b_ld = tr ? ldx : K;
    if (!make_map(&ta, a_ptr, a_rows, K, a_ld, BM) || !make_map(&tb, b_ptr, b_rows, K, b_ld, bn)) return BW_ERR_DRIVER;

    Epilogue ep;
    ep.out = out; ep.partial = splits > 1 ? workspace : nullptr; ep.bias = bias; ep.ldo = ldo;
    ep.out_type = out_type; ep.bias_type = bias_type; ep.accumulate = accumulate; ep.transposed = tr;
    ep.tokens = M; ep.features = N;
    dim3 grid(ceil_div(a_rows, BM), ceil_div(b_rows, bn), splits);
    int rc;
    switch (bn) {
        case 16: rc = launch<16>(ta, tb, ep, grid, kb_total, kb_per_split, s); break;
        case 32: rc = launch<32>(ta, tb, ep, grid, kb_total, kb_per_split, s); break;
        case 64: rc = launch<64>(ta, tb, ep, grid, kb_total, kb_per_split, s); break;
        case 128: rc = launch<128>(ta, tb, ep, grid, kb_total, kb_per_split, s); break;
        case 256: rc = launch<256>(ta, tb, ep, grid, kb_total, kb_per_split, s); break;
        default: return BW_ERR_BAD_ARG;
    }
    if (rc) return rc;
    if (splits > 1) {
        const size_t total = (size_t)M * N;
        const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
        splitk_reduce_kernel<<<blocks, 256, 0, s>>>(ep, splits);
        BW_LAUNCH_CHECK();
    }
    return 0;
}

// Reads and clears the status word (synchronises the device).  0: no wait ever gave up.
BW_EXPORT int bw_gemm_tc_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
    return v;
}
