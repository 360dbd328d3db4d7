// Paged causal grouped-query flash attention for prompt portions on the 5th-generation tensor
// cores (bfloat16, head size HEAD_DIM: a compile-time multiple of 64 up to 256).
//
// A CTA takes 128 stacked query rows (row = token * G + head-in-group: the G query heads of one
// kv head share every key and value tile) of one (request, kv head) and walks the keys in tiles
// of 64 up to the causal diagonal:
//   * TMA brings the query tile (3-D box: channels x heads x tokens) and, page by page through the
//     block table, the K and V tiles into 128-byte-swizzled shared memory (2 stages);
//   * S = Q K^T: tcgen05.mma (M 128, N 64) into one of two TMEM buffers, so that S of the next tile
//     is computed while the softmax warps work on this one;
//   * four softmax warps, one thread per row (no shuffles): tcgen05.ld of the row of S, mask,
//     maximum, then the probabilities 2^(s * scale - m) with running sum in float32, rounded to
//     bfloat16 pairs in the registers of the scores already used (the kernel stays within 128
//     registers) and written back with tcgen05.st over the first 32 columns of the S buffer;
//   * O += P V: tcgen05.mma with P read from tensor memory and V as an MN-major shared-memory
//     operand (keys are its K dimension), accumulated in TMEM over all tiles.  P has the two
//     buffers of S, so the softmax warps never wait for the P V of the tile before.  The
//     exponent's reference m follows the row maximum lazily: only when the maximum has grown by
//     more than 8 (a factor 256) since m was set does the warp wait for that P V and rescale its
//     rows of O in TMEM (tcgen05.ld, multiply, tcgen05.st); P stays below 2^8, the sums are
//     float32, and O / l at the end is the same quotient.
// Warp 4 issues the MMAs, warp 5 the TMA loads.  Keys past the request's length are never loaded
// (a resident page stands in, so the tile holds finite numbers) and are masked by position.
// Every wait is bounded and sets a status word.
#include "tcgen05.cuh"

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<multiple of 64>"
#endif
// 1 (the default): the MMA warp waits for the P V that reads a buffer before it issues the Q K^T that
// overwrites it.  0: it relies on tensor instructions of one thread running in issue order (measurement only).
#ifndef ATTN_STRICT_ORDER
#define ATTN_STRICT_ORDER 1
#endif

using bf16 = __nv_bfloat16;

namespace {

constexpr int HD = HEAD_DIM;
static_assert(HD % 64 == 0 && HD >= 64 && HD <= 256, "head size must be a multiple of 64 in [64, 256]");
constexpr int NS = HD / 64;            // 128-byte column slices of a row
constexpr int BM = 128, BN = 64, STAGES = 2;
constexpr int THREADS = 192;
constexpr int Q_SLICE = BM * 128, KV_SLICE = BN * 128;   // bytes of one column slice of a tile
constexpr int Q_BYTES = NS * Q_SLICE, KV_BYTES = NS * KV_SLICE;
constexpr int SMEM_BYTES = Q_BYTES + 2 * STAGES * KV_BYTES + 16 * 8 + 16;   // 2 CTAs per SM at head size 128
constexpr uint32_t TMEM_COLS = (128 + HD) <= 256 ? 256 : 512;   // S (two buffers of 64 columns), then O
constexpr uint32_t IDESC_QK = bw::umma_idesc_bf16(BM, BN, false);
constexpr uint32_t IDESC_PV = bw::umma_idesc_bf16(BM, HD, true);   // all channels in one product

__device__ int g_status = 0;

struct Params {
    bf16* out;
    const int* cu_q; const int* q_start; const int* kv_len; const int* block_table; const int* work;
    int max_blocks, nh, nkv, G, page_size, window, tpt;
    float scale_log2;
};

// 2^x, one MUFU instruction (the flush of denormal results to zero does not matter for softmax weights)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Two CTAs share an SM up to head size 128.  The bound is written for 256 threads, which caps the
// registers at 128 a thread: the six warps of a CTA lie unevenly on the SM's four register files
// (2, 2, 1, 1), and only with at most 128 registers does a new CTA fit beside a running one in
// whichever way its warps fall; with more, it started only once the SM was empty.
__global__ void __launch_bounds__(HD <= 128 ? 256 : THREADS, HD <= 128 ? 2 : 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, Params p) {
    BW_PDL_TRIGGER();
    extern __shared__ __align__(1024) uint8_t smem[];   // the swizzled tiles need 1024-byte alignment
    uint8_t* q_s = smem;
    uint8_t* k_s = q_s + Q_BYTES;                 // [STAGES][KV_BYTES]
    uint8_t* v_s = k_s + STAGES * KV_BYTES;
    uint64_t* bars = (uint64_t*)(v_s + STAGES * KV_BYTES);
    // 0 q_full, 1..2 k_full, 3..4 v_full, 5..6 k_empty, 7..8 v_empty, 9..10 s_full, 11..12 p_full, 13..14 pv_done:
    // one of each pair per S buffer, so that a wait by parity is never more than one phase behind
    uint32_t* tmem_slot = (uint32_t*)(bars + 16);
    const uint32_t bar0 = bw::smem_u32(bars);
    const uint32_t q_full = bar0, k_full = bar0 + 8, v_full = bar0 + 24, k_empty = bar0 + 40, v_empty = bar0 + 56,
                   s_full = bar0 + 72, p_full = bar0 + 88, pv_done = bar0 + 104;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        bw::mbar_init(q_full, 1);
        for (int s = 0; s < STAGES; ++s) {
            bw::mbar_init(k_full + 8 * s, 1); bw::mbar_init(v_full + 8 * s, 1); bw::mbar_init(k_empty + 8 * s, 1);
            bw::mbar_init(v_empty + 8 * s, 1); bw::mbar_init(s_full + 8 * s, 1);
            bw::mbar_init(p_full + 8 * s, 4); bw::mbar_init(pv_done + 8 * s, 1);
        }
        bw::fence_barrier_init();
        bw::tma_prefetch_desc(&tmQ); bw::tma_prefetch_desc(&tmK); bw::tma_prefetch_desc(&tmV);
        tmem_slot[1] = (uint32_t)g_status;
    }
    if (warp == 4) bw::tmem_alloc(bw::smem_u32(tmem_slot), TMEM_COLS);
    bw::tc_fence_before();
    __syncthreads();
    bw::tc_fence_after();
    BW_PDL_WAIT();   // queries, keys and values of this step come from the kernels before
    const uint32_t tmem_base = *tmem_slot;
    const bool dead = tmem_slot[1] != 0;
    const uint32_t tmem_S = tmem_base, tmem_O = tmem_base + 128;   // S buffer b at tmem_S + 64 b

    // the kv heads of one work item are neighbours in the launch order, so the items (longest first)
    // start in that order across all heads
    const int4 wk = reinterpret_cast<const int4*>(p.work)[blockIdx.x / p.nkv];
    const int r = wk.x, tok0 = wk.y, g = blockIdx.x % p.nkv;
    const int q_len = p.cu_q[r + 1] - p.cu_q[r];
    const int kv_len = p.kv_len[r];
    const int ntok = min(p.tpt, q_len - tok0);
    const int n_rows = ntok * p.G;
    const int q_pos0 = p.q_start[r] + tok0;
    const int last_pos = q_pos0 + ntok - 1;
    const int first_key = p.window > 0 ? max(0, q_pos0 - p.window + 1) : 0;
    const int t_lo = first_key / BN, n_tiles = last_pos / BN - t_lo + 1;
    const int* bt = p.block_table + (size_t)r * p.max_blocks;

    if (dead) {
        // an earlier launch timed out: do nothing
    } else if (warp == 5) {
        if (lane == 0) {
            // queries: one 3-D box per column slice (channels x the G heads of this kv head x tokens)
            bw::mbar_expect_tx(q_full, NS * p.G * p.tpt * 128);
#pragma unroll
            for (int h = 0; h < NS; ++h)
                bw::tma_load_3d(bw::smem_u32(q_s + h * Q_SLICE), &tmQ, q_full, h * 64, g * p.G, p.cu_q[r] + tok0);
        }
        // Lane pg owns page pg of every tile: its page id is looked up one tile ahead (the lookup's
        // latency is off the path) and its boxes are issued beside the other lanes'.
        const int ppt = BN / p.page_size;   // pages per tile
        auto lookup = [&](int i) {
            const int key = (t_lo + i) * BN + lane * p.page_size;
            int page = (lane < ppt && i < n_tiles && key < kv_len) ? bt[key / p.page_size] : -1;
            return page < 0 ? 0 : page;      // never read: a resident page keeps the tile finite
        };
        // Keys and values have stages of their own: a key stage is free as soon as Q K^T of the tile
        // before last has run, a value stage only after its P V, so the keys run one tile ahead of
        // the values and neither load is waited for in the steady state.
        auto load = [&](const CUtensorMap* tm, uint8_t* base, uint32_t full, int i, int page) {
            const int s = i & 1;
            if (lane == 0) bw::mbar_expect_tx(full + 8 * s, KV_BYTES);
            __syncwarp();
            if (lane < ppt) {
                const int y = (page * p.nkv + g) * p.page_size;
                const uint32_t off = s * KV_BYTES + lane * p.page_size * 128;
#pragma unroll
                for (int h = 0; h < NS; ++h)
                    bw::tma_load_2d(bw::smem_u32(base + off + h * KV_SLICE), tm, full + 8 * s, h * 64, y);
            }
        };
        int page_v = lookup(0), page_k = lookup(1);
        load(&tmK, k_s, k_full, 0, page_v);
        for (int i = 0; i < n_tiles; ++i) {
            const int pk = page_k, pv = page_v;
            page_v = pk; page_k = lookup(i + 2);
            if (i + 1 < n_tiles) {   // keys of tile i + 1
                if (i >= 1 && !__all_sync(0xffffffffu, bw::mbar_wait(k_empty + 8 * ((i + 1) & 1), ((i - 1) >> 1) & 1, &g_status, 15))) break;
                load(&tmK, k_s, k_full, i + 1, pk);
            }
            if (i >= 2 && !__all_sync(0xffffffffu, bw::mbar_wait(v_empty + 8 * (i & 1), ((i - 2) >> 1) & 1, &g_status, 19))) break;
            load(&tmV, v_s, v_full, i, pv);
        }
    } else if (warp == 4) {
        if (lane == 0) {
            auto issue_qk = [&](int s) {   // keys of stage s -> S buffer s
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    const uint64_t da = bw::umma_smem_desc_sw128(bw::smem_u32(q_s + (ks >> 2) * Q_SLICE)) + 2 * (ks & 3);
                    const uint64_t db = bw::umma_smem_desc_sw128(bw::smem_u32(k_s + s * KV_BYTES + (ks >> 2) * KV_SLICE)) + 2 * (ks & 3);
                    bw::umma_bf16(tmem_S + 64 * s, da, db, IDESC_QK, ks != 0);
                }
                bw::umma_commit(s_full + 8 * s);
                bw::umma_commit(k_empty + 8 * s);
            };
            auto issue_pv = [&](int s, bool first) {   // P in the first 32 columns of S buffer s, values of stage s
                // one product per 16 keys over all HD channels: the operand's 64-channel slices lie
                // KV_SLICE bytes apart (the descriptor's leading byte offset)
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk) {
                    const uint64_t db = bw::umma_smem_desc_mn_sw128(bw::smem_u32(v_s + s * KV_BYTES), KV_SLICE)
                                        + (uint64_t)kk * (2048 >> 4);   // 16 keys = two 8-row groups
                    bw::umma_bf16_ts(tmem_O, tmem_S + 64 * s + 8 * kk, db, IDESC_PV, !(first && kk == 0));
                }
                bw::umma_commit(pv_done + 8 * s);
                bw::umma_commit(v_empty + 8 * s);
            };
            bool ok = bw::mbar_wait(q_full, 0, &g_status, 11) && bw::mbar_wait(k_full, 0, &g_status, 12);
            if (ok) { bw::tc_fence_after(); issue_qk(0); }
            for (int i = 0; i < n_tiles && ok; ++i) {
                const int s = i & 1;
                if (i + 1 < n_tiles) {
                    // S of the next tile, while the softmax warps work on this one.  Its buffer holds
                    // P of tile i - 1, which the P V issued before still reads as its operand: that
                    // product must be complete before this one may overwrite the buffer (the order of
                    // two tensor instructions is promised only when they write the same accumulator).
                    if (!bw::mbar_wait(k_full + 8 * (s ^ 1), ((i + 1) >> 1) & 1, &g_status, 14)) break;
#if ATTN_STRICT_ORDER
                    if (i >= 1 && !bw::mbar_wait(pv_done + 8 * (s ^ 1), ((i - 1) >> 1) & 1, &g_status, 22)) break;
#endif
                    bw::tc_fence_after();
                    issue_qk(s ^ 1);
                }
                if (!bw::mbar_wait(p_full + 8 * s, (i >> 1) & 1, &g_status, 13)) break;   // P(i) written, O rescaled
                if (!bw::mbar_wait(v_full + 8 * s, (i >> 1) & 1, &g_status, 20)) break;
                bw::tc_fence_after();
                issue_pv(s, i == 0);
            }
        }
    } else {
        const int row = warp * 32 + lane;
        const bool row_ok = row < n_rows;
        const int tok = row / p.G, hg = row - tok * p.G;
        const int qpos = q_pos0 + tok;
        const int lo = p.window > 0 ? max(0, qpos - p.window + 1) : 0;
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        float m = -INFINITY, l = 0.f;   // m: the reference of the exponents (at most 8 below the row maximum)
        bool ok = true;

        for (int i = 0; i < n_tiles; ++i) {
            if (!__all_sync(0xffffffffu, bw::mbar_wait(s_full + 8 * (i & 1), (i >> 1) & 1, &g_status, 16))) { ok = false; break; }
            bw::tc_fence_after();
            const int key0 = (t_lo + i) * BN;
            const bool need_mask = !row_ok || (key0 + BN - 1 > q_pos0) || (p.window > 0 && key0 < last_pos - p.window + 1);
            // The row of S, unscaled (scale > 0, so the maximum commutes with it; masked keys become -inf).
            // It stays in these 64 registers; the packed probabilities take the place of the first 32
            // as they are made, so that the kernel stays within 128 registers (see the launch bounds).
            const uint32_t s_row = tmem_S + 64 * (i & 1) + lane_base;
            uint32_t v[BN];
            bw::tmem_ld_32x32(s_row, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
            bw::tmem_ld_32x32(s_row + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
            bw::tmem_ld_wait();
            if (need_mask) {   // one branch per tile, not one per key
#pragma unroll
                for (int c = 0; c < BN; ++c) {
                    const int kp = key0 + c;
                    if (!row_ok || kp > qpos || kp < lo) v[c] = 0xff800000u;   // -inf
                }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < BN; c += 2)   // max(m, a, b): one three-input instruction where the hardware has it
                mx4[(c >> 1) & 3] = fmaxf(mx4[(c >> 1) & 3], fmaxf(__uint_as_float(v[c]), __uint_as_float(v[c + 1])));
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
            const bool grow = mx > m + 8.f;   // also the first finite maximum of a row (m is -inf until then)
            float factor = 1.f;
            if (grow) {
                if (m != -INFINITY) factor = fast_exp2(m - mx);
                l *= factor;
                m = mx;
            }
            if (i > 0 && __any_sync(0xffffffffu, grow)) {
                // O may be read once the P V of the tile before is done (the P V of tile i - 3, the one
                // before on that barrier, is: S of this tile was computed after the P V of tile i - 2)
                if (!__all_sync(0xffffffffu, bw::mbar_wait(pv_done + 8 * ((i - 1) & 1), ((i - 1) >> 1) & 1, &g_status, 17))) { ok = false; break; }
                bw::tc_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < HD; c0 += 16) {   // rare: a rolled loop of small pieces, few registers
                    uint32_t o[16];
                    bw::tmem_ld_32x16(tmem_O + lane_base + c0, o);
                    bw::tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 16; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * factor);
                    bw::tmem_st_32x16(tmem_O + lane_base + c0, o);
                }
                bw::tmem_st_wait();
            }
            const float mu = m == -INFINITY ? 0.f : m;
            // The probabilities 2^(s * scale - mu), rounded to bfloat16 pairs: pair c / 2 goes where score
            // c / 2 was (already used), and the 32 pairs over the first 32 columns of the row of S.
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < BN; c += 2) {
                const float p0 = fast_exp2(fmaf(__uint_as_float(v[c]), p.scale_log2, -mu));
                const float p1 = fast_exp2(fmaf(__uint_as_float(v[c + 1]), p.scale_log2, -mu));
                sum4[(c >> 1) & 3] += p0 + p1;
                v[c >> 1] = pack_bf16(p0, p1);
            }
            bw::tmem_st_32x32(s_row, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
            l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            // Values of keys that do not exist (past the request's length, or on a page the block
            // table no longer holds) are whatever the stand-in page contained: zero them, since a
            // probability of 0 times a stale NaN would still be NaN.  Rare: the last tile, a window's edge.
            if (key0 + BN > kv_len || (p.window > 0 && key0 < first_key)) {
                if (!__all_sync(0xffffffffu, bw::mbar_wait(v_full + 8 * (i & 1), (i >> 1) & 1, &g_status, 21))) { ok = false; break; }
                for (int pg = 0; pg < BN / p.page_size; ++pg) {
                    const int pkey = key0 + pg * p.page_size;
                    int bad_from = p.page_size;   // first row of this page to clear
                    if (pkey >= kv_len || bt[pkey / p.page_size] < 0) bad_from = 0;
                    else if (pkey + p.page_size > kv_len) bad_from = kv_len - pkey;
                    const int n_bad = p.page_size - bad_from;
                    uint8_t* vbase = v_s + (i & 1) * KV_BYTES + (pg * p.page_size + bad_from) * 128;
                    for (int idx = row; idx < n_bad * NS * 8; idx += BM) {
                        const int rk = idx / (NS * 8), rem = idx - rk * (NS * 8);
                        *reinterpret_cast<uint4*>(vbase + (rem >> 3) * KV_SLICE + rk * 128 + (rem & 7) * 16) = make_uint4(0, 0, 0, 0);
                    }
                }
                bw::fence_proxy_async_smem();
            }
            bw::tmem_st_wait();
            bw::tc_fence_before();
            __syncwarp();
            if (lane == 0) bw::mbar_arrive(p_full + 8 * (i & 1));
        }
        if (ok) ok = __all_sync(0xffffffffu, bw::mbar_wait(pv_done + 8 * ((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1, &g_status, 18));
        if (ok) {
            bw::tc_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            bf16* dst = p.out + ((size_t)(p.cu_q[r] + tok0 + tok) * p.nh + g * p.G + hg) * HD;
#pragma unroll
            for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t v[32];
                bw::tmem_ld_32x32(tmem_O + lane_base + c0, v);
                bw::tmem_ld_wait();
                if (row_ok) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        *reinterpret_cast<uint4*>(dst + c0 + c) =
                            make_uint4(pack_bf16(__uint_as_float(v[c]) * inv, __uint_as_float(v[c + 1]) * inv),
                                       pack_bf16(__uint_as_float(v[c + 2]) * inv, __uint_as_float(v[c + 3]) * inv),
                                       pack_bf16(__uint_as_float(v[c + 4]) * inv, __uint_as_float(v[c + 5]) * inv),
                                       pack_bf16(__uint_as_float(v[c + 6]) * inv, __uint_as_float(v[c + 7]) * inv));
                    }
                }
            }
        }
    }
    bw::tc_fence_before();
    __syncthreads();
    if (warp == 4) bw::tmem_dealloc(tmem_base, TMEM_COLS);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = (EncodeTiledFn)ptr;
    }
    return fn;
}

bool encode(CUtensorMap* m, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
            const cuuint32_t* box) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

BW_EXPORT int bw_attention_tc_head_dim() { return HD; }

// Whether this kernel takes the geometry: pages of 8, 16, 32 or 64 tokens, at most 128 query heads
// per kv head, 16-byte aligned tensors.
BW_EXPORT int bw_attention_tc_supported(int nh, int nkv, int page_size) {
    if (nkv <= 0 || nh % nkv) return 0;
    const int G = nh / nkv;
    return (G <= 128 && page_size >= 8 && page_size <= 64 && 64 % page_size == 0) ? 1 : 0;
}

// work: n_items int4 (request, first token of the 128-row tile within the request's segment, 0, 0);
// a tile holds 128 / G tokens.  q, out: [T, nh * HD] bf16; pages: [num_pages, nkv, page_size, HD] bf16.
BW_EXPORT int bw_attention_tc(const void* q, const void* k_pages, const void* v_pages, void* out, const int* cu_q,
                              const int* q_start, const int* kv_len, const int* block_table, int max_blocks,
                              const int* work, int n_items, int T, int nh, int nkv, int page_size, int num_pages,
                              int window, float scale, void* stream) {
    if (n_items <= 0) return 0;
    if (!bw_attention_tc_supported(nh, nkv, page_size) || !(scale > 0.f)) return BW_ERR_UNSUPPORTED;
    if ((((uintptr_t)q | (uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)out) & 15) != 0) return BW_ERR_UNSUPPORTED;
    const int G = nh / nkv, tpt = BM / G;
    CUtensorMap tq, tk, tv;
    {
        cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)nh, (cuuint64_t)T};
        cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)nh * HD * 2};
        cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)tpt};
        if (!encode(&tq, q, 3, dims, strides, box)) return BW_ERR_DRIVER;
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)num_pages * nkv * page_size};
        cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)page_size};
        if (!encode(&tk, k_pages, 2, dims, strides, box) || !encode(&tv, v_pages, 2, dims, strides, box)) return BW_ERR_DRIVER;
    }
    static bool attr_done[bw::MAX_DEVICES];
    if (cudaError_t e = bw::allow_dynamic_smem(attn_tc_kernel, SMEM_BYTES, attr_done); e != cudaSuccess) return (int)e;
    Params p;
    p.out = (bf16*)out; p.cu_q = cu_q; p.q_start = q_start; p.kv_len = kv_len; p.block_table = block_table;
    p.work = work; p.max_blocks = max_blocks; p.nh = nh; p.nkv = nkv; p.G = G; p.page_size = page_size;
    p.window = window > 0 ? window : 0; p.tpt = tpt;
    p.scale_log2 = scale * 1.4426950408889634f;
    bw::launch((attn_tc_kernel), dim3((unsigned)n_items * nkv), dim3(THREADS), SMEM_BYTES, (cudaStream_t)stream, tq, tk, tv, p);
    BW_LAUNCH_CHECK();
    return 0;
}


BW_EXPORT int bw_attention_tc_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
    return v;
}
