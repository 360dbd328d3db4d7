// bfloat16 matrix product on the 5th-generation tensor cores:
//     acc[i, j] = sum_k A[i, k] * B[j, k]      (A: [Ra, K], B: [Rb, K], both row-major)
// A persistent kernel: one CTA per SM walks a list of work items (output tile, K split).
// TMA brings 128 x 64 tiles of A and BN x 64 tiles of B into a shared-memory ring (128-byte
// swizzle), one elected thread issues tcgen05.mma into one of TWO TMEM accumulators, and
// four epilogue warps drain the other one with tcgen05.ld, so the epilogue of an item
// overlaps the main loop of the next.  Each CTA loads its own tiles (no multicast).
//
// The same kernel serves both orientations of  out[tokens, features] = x . w^T:
//   normal     A = x (tokens),   B = w (features): prefill, many tokens;
//   transposed A = w (features), B = x (tokens):   few tokens (decode): the weight
//              rows fill the 128-row MMA dimension and the tokens are the narrow N.
// Split-K: every item writes its float32 partial tile to scratch; per (tile, 32-row
// quarter) a counter tells the warp that finishes last to add the partials IN SPLIT
// ORDER (deterministic) and run the epilogue.  Counters return to zero by themselves.
// Epilogue: + bias[feature], then store float32 | bfloat16, or add into float32 out
// (the residual stream), or SwiGLU over interleaved gate/up features -> bfloat16, or rotary
// position encoding of a fused q/k/v projection with the keys and values written to their pages.
//
// With 512 tokens or more and no K split the product runs on CTA PAIRS instead
// (gemm_pair_kernel, cta_group::2): two CTAs of a cluster share a tile of 256 tokens, each loads
// half of the weight tile, and the leader's MMAs read both CTAs' shared memory.
//
// Roles (192 threads): warp 0 TMA producer, warp 1 TMEM owner + MMA issuer, warps
// 2..5 epilogue (TMEM lane quarter = warp % 4).  Every wait is bounded; a timeout sets
// the status word and all roles fall through to the common exit where TMEM is freed.
#include <cstring>
#include "tcgen05.cuh"

using bf16 = __nv_bfloat16;

namespace {

constexpr int BM = 128;       // rows of the A tile = MMA M
constexpr int BK = 64;        // k-block: 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;
constexpr int THREADS = 192;
// Epilogue staging, per epilogue warp a 32 x 33 float block or two 32 x 32 boxes for TMA.  Only the normal
// orientation uses it, and that has tiles of 128 columns or more: the narrow kernels do without.
template <int BN> __host__ __device__ constexpr int staging_bytes() { return BN >= 128 ? 4 * 2 * 4096 : 0; }
constexpr int SMEM_BUDGET = 226 * 1024 - staging_bytes<256>() - 2048;
constexpr int FUSED_REDUCE_MAX_TOKENS = 16;   // split-K sums inside the kernel up to this many tokens
constexpr int SWIGLU_BLOCK = 16;   // gate/up features are interleaved in blocks of 16 rows of the weight
#ifndef GEMM_NARROW_STAGES
#define GEMM_NARROW_STAGES 8       // stages of the ring of the kernel for up to 16 tokens
#endif
#ifndef GEMM_NARROW_CTAS
#define GEMM_NARROW_CTAS 1         // CTAs of that kernel the register allocation leaves room for on an SM
#endif

__device__ int g_status = 0;  // 0 ok; else the code of the first wait that gave up
int g_pair_mode = -1;         // see bw_gemm_tc_pair_mode

// Rotary epilogue of a fused q/k/v projection: features are (q heads, k heads, v heads) x hd.  In
// the rotated heads the weight rows are ordered so that features 2j and 2j + 1 are channel j and
// its partner j + rd / 2: a lane finds the partner in its neighbour.  Queries go to q_out
// [tokens, nh * hd]; keys and values to the page of the token's position
// ([num_pages, nkv, page_size, hd]) that kv_slot names; without kv_slot no keys or values are written.
struct RopeOut {
    const float* table;          // [tokens, rd]: cos (rd / 2), then sin (rd / 2) of the token's angles
    const int* kv_slot;          // [tokens]: page * page_size + slot of the token's position, -1: none; null: no append
    bf16* q_out; bf16* k_pages; bf16* v_pages;
    int nh, nkv, hd, rd, page_size;
};

struct Epilogue {
    void* out;            // [tokens, features] (SwiGLU: [tokens, features / 2]), row stride ldo (elements)
    float* partial;       // split-K: [splits, tokens, features] dense float32; else null
    int* counters;        // split-K: one per (tile, quarter), zero before and after the launch
    const void* bias;     // [features] or null
    long long ldo;
    int out_type, bias_type, accumulate, transposed, swiglu;
    int tokens, features, splits;
    int rope_on;
    int tma_add;          // normal orientation, out += : 32 x 32 boxes go out through the tensor map tmC
    int stream;           // the k-blocks of all tiles, laid end to end, are cut into one equal range per CTA
    int planes;           // split-K: the partial planes ARE the result (the bias in plane 0); whoever reads them adds them up
    RopeOut rope;
};

__device__ __forceinline__ float bias_at(const Epilogue& ep, int feature) {
    if (!ep.bias) return 0.f;
    return ep.bias_type == BW_F32 ? ((const float*)ep.bias)[feature] : __bfloat162float(((const bf16*)ep.bias)[feature]);
}

// Where the rotary epilogue puts feature `feature` of a token: the head, the channel within it,
// whether it is rotated and the sign of its partner's sine.
struct RopeSlot { int head, channel, j; bool rot, second; };
__device__ __forceinline__ RopeSlot rope_slot(const RopeOut& ro, int feature) {
    RopeSlot s;
    s.head = feature / ro.hd;
    const int li = feature - s.head * ro.hd;
    s.rot = s.head < ro.nh + ro.nkv && li < ro.rd;
    s.j = li >> 1; s.second = (li & 1) != 0;
    s.channel = s.rot ? s.j + (s.second ? (ro.rd >> 1) : 0) : li;
    return s;
}

// row of the pages ([page, kv head, slot]) where a key / value of kv head `kvh` goes, from the token's
// kv_slot value (page * page_size + slot), or -1
__device__ __forceinline__ long long rope_page_row(const RopeOut& ro, int kv_slot, int kvh) {
    if (kv_slot < 0) return -1;
    const int page = kv_slot / ro.page_size;
    return ((long long)page * ro.nkv + kvh) * ro.page_size + (kv_slot - page * ro.page_size);
}

// cosine and signed sine of a rotated channel (first half: x cos - partner sin; second: x cos + partner sin)
__device__ __forceinline__ float2 rope_angle(const RopeOut& ro, const RopeSlot& sl, int token) {
    if (!sl.rot) return make_float2(1.f, 0.f);
    const float cs = __ldg(ro.table + (size_t)token * ro.rd + sl.j);
    const float sn = __ldg(ro.table + (size_t)token * ro.rd + (ro.rd >> 1) + sl.j);
    return make_float2(cs, sl.second ? sn : -sn);
}

__device__ __forceinline__ void rope_store(const RopeOut& ro, const RopeSlot& sl, int token, long long page_row,
                                           float2 angle, float x, float partner) {
    const float y = sl.rot ? x * angle.x + partner * angle.y : x;
    if (sl.head < ro.nh) {
        ro.q_out[((size_t)token * ro.nh + sl.head) * ro.hd + sl.channel] = __float2bfloat16_rn(y);
    } else if (page_row >= 0) {
        bf16* pages = sl.head < ro.nh + ro.nkv ? ro.k_pages : ro.v_pages;
        pages[(size_t)page_row * ro.hd + sl.channel] = __float2bfloat16_rn(y);
    }
}

template <int BN> __host__ __device__ constexpr int stages_for() {
    constexpr int per = A_BYTES + BN * BK * 2;
    constexpr int s = SMEM_BUDGET / per;
    // The narrowest tile (decode with up to 16 tokens): 8 stages of 18 KB.  A CTA streams what its
    // stages hold in flight over the latency of a load (about 2 us from DRAM): 5 stages drew about
    // 40 GB/s, less than an SM's share of the bandwidth.  Measured on a decode step at batch 8 and
    // context 8,192 (ms): 5 stages 5.08, 6: 4.94, 7: 4.93, 8: 4.91, 10: 4.95, 12: 5.02.  (With 5
    // stages two CTAs fit on an SM and the next product's CTAs could request weights while this
    // one's drained; the deeper ring is worth more.)
    return BN <= 16 ? GEMM_NARROW_STAGES : (s > 8 ? 8 : s);
}

// The rotary epilogue of G consecutive tokens of one feature (one lane), in two halves: what does
// not depend on the sums (the tokens' cache slots and angles) is fetched first, so a caller that
// still has sums to form can overlap the two.
template <int G> struct RopeCtx { RopeSlot sl; float b, bp; int kvh; int kv[G]; float2 ang[G]; };

template <int G>
__device__ __forceinline__ void rope_prefetch(const Epilogue& ep, RopeCtx<G>& cx, int token0, int nvalid,
                                              int feature, bool fvalid) {
    const RopeOut& ro = ep.rope;
    cx.sl = rope_slot(ro, fvalid ? feature : 0);
    cx.b = fvalid ? bias_at(ep, feature) : 0.f;
    cx.bp = fvalid ? bias_at(ep, feature ^ 1) : 0.f;   // the partner's (the feature count is even)
    cx.kvh = cx.sl.head < ro.nh + ro.nkv ? cx.sl.head - ro.nh : cx.sl.head - ro.nh - ro.nkv;
    const bool paged = fvalid && cx.sl.head >= ro.nh && ro.kv_slot;
#pragma unroll
    for (int k = 0; k < G; ++k) {
        const bool live = k < nvalid && fvalid;
        cx.kv[k] = (paged && live) ? __ldg(ro.kv_slot + token0 + k) : -1;
        cx.ang[k] = live ? rope_angle(ro, cx.sl, token0 + k) : make_float2(1.f, 0.f);
    }
}

template <int G>
__device__ __forceinline__ void rope_finish(const Epilogue& ep, const RopeCtx<G>& cx, const float* vals, int token0,
                                            int nvalid, bool fvalid) {
#pragma unroll
    for (int k = 0; k < G; ++k) {
        const float partner = __shfl_xor_sync(0xffffffffu, vals[k], 1) + cx.bp;
        if (k < nvalid && fvalid)
            rope_store(ep.rope, cx.sl, token0 + k, rope_page_row(ep.rope, cx.kv[k], cx.kvh), cx.ang[k], vals[k] + cx.b, partner);
    }
}

// stages of the pair kernel: a stage holds 128 rows of x and BN / 2 rows of w
template <int BN> __host__ __device__ constexpr int pair_stages() {
    constexpr int per = A_BYTES + (BN / 2) * BK * 2;
    constexpr int s = SMEM_BUDGET / per;
    return s > 8 ? 8 : s;
}

// The lane holds the finished sums vals[0..N) of ONE feature for N consecutive tokens (token0 + c);
// the 32 lanes of the warp hold 32 consecutive features.  nvalid (the same in all lanes) of the
// tokens exist.  When the result is added to `out`, all old values are fetched before the first
// store, so the loads are in flight together instead of one round trip per token.
template <int N, bool ROPE>
__device__ __forceinline__ void emit(const Epilogue& ep, float* part, const float (&vals)[N], int token0,
                                     int nvalid, int feature, bool fvalid) {
    if (part) {
        const float b = (ep.planes && part == ep.partial && fvalid) ? bias_at(ep, feature) : 0.f;
#pragma unroll
        for (int c = 0; c < N; ++c)
            if (c < nvalid && fvalid) part[(size_t)(token0 + c) * ep.features + feature] = vals[c] + b;
        return;
    }
    if (ep.swiglu) {
        // lanes 0..15 hold gate, lanes 16..31 up of the same 16 output features
        const int lane = threadIdx.x & 31;
        const int j = (feature / (2 * SWIGLU_BLOCK)) * SWIGLU_BLOCK + lane;
#pragma unroll
        for (int c = 0; c < N; ++c) {
            const float other = __shfl_xor_sync(0xffffffffu, vals[c], 16);
            if (c < nvalid && fvalid && lane < SWIGLU_BLOCK)
                ((bf16*)ep.out)[(size_t)(token0 + c) * ep.ldo + j] =
                    __float2bfloat16_rn(__fdividef(vals[c], 1.f + __expf(-vals[c])) * other);
        }
        return;
    }
    if constexpr (ROPE) {
        // eight tokens at a time: their cache slots and angles are fetched before the first store
        constexpr int G = N < 8 ? N : 8;
#pragma unroll
        for (int c0 = 0; c0 < N; c0 += G) {
            RopeCtx<G> cx;
            rope_prefetch<G>(ep, cx, token0 + c0, nvalid - c0, feature, fvalid);
            rope_finish<G>(ep, cx, &vals[c0], token0 + c0, nvalid - c0, fvalid);
        }
        return;
    }
    if (!fvalid) return;
    const float b = bias_at(ep, feature);
    const size_t off = (size_t)token0 * ep.ldo + feature;
    if (ep.out_type == BW_F32) {
        float* o = (float*)ep.out + off;
        float old[N];
        if (ep.accumulate) {
#pragma unroll
            for (int c = 0; c < N; ++c) old[c] = c < nvalid ? o[(size_t)c * ep.ldo] : 0.f;
        }
#pragma unroll
        for (int c = 0; c < N; ++c)
            if (c < nvalid) o[(size_t)c * ep.ldo] = vals[c] + b + (ep.accumulate ? old[c] : 0.f);
    } else {
        bf16* o = (bf16*)ep.out + off;
#pragma unroll
        for (int c = 0; c < N; ++c)
            if (c < nvalid) o[(size_t)c * ep.ldo] = __float2bfloat16_rn(vals[c] + b);
    }
}

// Rotary epilogue in the normal orientation: the thread holds 32 consecutive features f0 .. f0 + 31
// (the first n_features of them belong to this tile; a multiple of 16) of ONE token (v, float32 bits straight from TMEM).  Partners are neighbours in its registers, the
// cache slot of the token is read once per tile (kv_slot < 0: no keys and values are written), and
// every store is 16 bytes when rd is a multiple of 16.
__device__ __forceinline__ void rope_direct(const Epilogue& ep, const uint32_t (&v)[32], int token, int f0,
                                         int n_features, int kv_slot) {
    const RopeOut& ro = ep.rope;
    const int half = ro.rd >> 1;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int fh = f0 + 16 * h;
        if (fh >= ep.features || 16 * h >= n_features) break;
        const int head = fh / ro.hd, li0 = fh - head * ro.hd;
        bf16* dst;
        if (head < ro.nh) dst = ro.q_out + ((size_t)token * ro.nh + head) * ro.hd;
        else {
            if (kv_slot < 0) continue;
            const bool is_k = head < ro.nh + ro.nkv;
            const int kvh = is_k ? head - ro.nh : head - ro.nh - ro.nkv;
            dst = (is_k ? ro.k_pages : ro.v_pages) + (size_t)rope_page_row(ro, kv_slot, kvh) * ro.hd;
        }
        float x[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) x[i] = __uint_as_float(v[16 * h + i]) + bias_at(ep, fh + i);
        const bool rotated_head = head < ro.nh + ro.nkv;
        if ((ro.rd & 15) == 0) {
            if (rotated_head && li0 < ro.rd) {
                const int j0 = li0 >> 1;
                const float4* tc = reinterpret_cast<const float4*>(ro.table + (size_t)token * ro.rd + j0);
                const float4* ts = reinterpret_cast<const float4*>(ro.table + (size_t)token * ro.rd + half + j0);
                const float4 c0 = __ldg(tc), c1 = __ldg(tc + 1), s0 = __ldg(ts), s1 = __ldg(ts + 1);
                const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
                float lo[8], hi[8];
#pragma unroll
                for (int p = 0; p < 8; ++p) {
                    lo[p] = x[2 * p] * cs[p] - x[2 * p + 1] * sn[p];
                    hi[p] = x[2 * p + 1] * cs[p] + x[2 * p] * sn[p];
                }
                *reinterpret_cast<uint4*>(dst + j0) = make_uint4(bw::pack_bf16x2(lo[0], lo[1]), bw::pack_bf16x2(lo[2], lo[3]),
                                                                 bw::pack_bf16x2(lo[4], lo[5]), bw::pack_bf16x2(lo[6], lo[7]));
                *reinterpret_cast<uint4*>(dst + j0 + half) = make_uint4(bw::pack_bf16x2(hi[0], hi[1]), bw::pack_bf16x2(hi[2], hi[3]),
                                                                        bw::pack_bf16x2(hi[4], hi[5]), bw::pack_bf16x2(hi[6], hi[7]));
            } else {
                *reinterpret_cast<uint4*>(dst + li0) = make_uint4(bw::pack_bf16x2(x[0], x[1]), bw::pack_bf16x2(x[2], x[3]),
                                                                  bw::pack_bf16x2(x[4], x[5]), bw::pack_bf16x2(x[6], x[7]));
                *reinterpret_cast<uint4*>(dst + li0 + 8) = make_uint4(bw::pack_bf16x2(x[8], x[9]), bw::pack_bf16x2(x[10], x[11]),
                                                                      bw::pack_bf16x2(x[12], x[13]), bw::pack_bf16x2(x[14], x[15]));
            }
        } else {
#pragma unroll
            for (int p = 0; p < 8; ++p) {
                const int li = li0 + 2 * p;
                if (rotated_head && li < ro.rd) {
                    const int j = li >> 1;
                    const float cs = __ldg(ro.table + (size_t)token * ro.rd + j);
                    const float sn = __ldg(ro.table + (size_t)token * ro.rd + half + j);
                    dst[j] = __float2bfloat16_rn(x[2 * p] * cs - x[2 * p + 1] * sn);
                    dst[j + half] = __float2bfloat16_rn(x[2 * p + 1] * cs + x[2 * p] * sn);
                } else {
                    dst[li] = __float2bfloat16_rn(x[2 * p]);
                    dst[li + 1] = __float2bfloat16_rn(x[2 * p + 1]);
                }
            }
        }
    }
}

// SwiGLU epilogue in the normal orientation: the thread holds 32 consecutive features f0 .. f0 + 31 of
// ONE token, f0 a multiple of 32: 16 gate sums, then the 16 up sums of the same output features.
// It writes silu(gate) * up for those 16 features as 32 contiguous bytes.
__device__ __forceinline__ void swiglu_direct(const Epilogue& ep, const uint32_t (&v)[32], int token, int f0) {
    float y[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float g = __uint_as_float(v[i]), u = __uint_as_float(v[16 + i]);
        y[i] = __fdividef(g, 1.f + __expf(-g)) * u;
    }
    bf16* dst = (bf16*)ep.out + (size_t)token * ep.ldo + (f0 / (2 * SWIGLU_BLOCK)) * SWIGLU_BLOCK;
    if ((ep.ldo & 7) == 0 && ((uintptr_t)ep.out & 15) == 0) {
        *reinterpret_cast<uint4*>(dst) = make_uint4(bw::pack_bf16x2(y[0], y[1]), bw::pack_bf16x2(y[2], y[3]),
                                                    bw::pack_bf16x2(y[4], y[5]), bw::pack_bf16x2(y[6], y[7]));
        *reinterpret_cast<uint4*>(dst + 8) = make_uint4(bw::pack_bf16x2(y[8], y[9]), bw::pack_bf16x2(y[10], y[11]),
                                                        bw::pack_bf16x2(y[12], y[13]), bw::pack_bf16x2(y[14], y[15]));
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) dst[i] = __float2bfloat16_rn(y[i]);
    }
}

// The work items of one CTA, the same sequence in each of its roles.
//   classic: item w = blockIdx.x + k * gridDim.x is (tile w % tiles, K split w / tiles);
//   stream:  the k-blocks of all tiles are laid end to end and the CTA owns the range
//            [c * total / G, (c + 1) * total / G), cut where it crosses a tile.  Every SM then
//            streams the same number of bytes however the tiles divide among the SMs.  A tile that
//            two CTAs share is summed like a K split: part = the CTA's rank among them.  (A range
//            is at least one tile long, the host sees to that, so no tile has more than two parts.)
struct Item { int tile, kb0, nkb, part, nparts; };
struct Items {
    int kb_total, kb_per_split, tiles, num_work, splits, stream, w, stride;
    long long lo, hi, total;
    // first, stride: the CTA's place among the CTAs (or CTA pairs) that share the items; default: the grid
    __device__ Items(const Epilogue& ep, int kb_total_, int kb_per_split_, int tiles_, int num_work_, int first = -1,
                     int stride_ = 0)
        : kb_total(kb_total_), kb_per_split(kb_per_split_), tiles(tiles_), num_work(num_work_), splits(ep.splits),
          stream(ep.stream), w(first < 0 ? (int)blockIdx.x : first), stride(stride_ > 0 ? stride_ : (int)gridDim.x) {
        total = (long long)tiles * kb_total;
        lo = (long long)blockIdx.x * total / gridDim.x;
        hi = (long long)(blockIdx.x + 1) * total / gridDim.x;
    }
    __device__ int owner(long long kb) const {   // the CTA whose range holds k-block kb
        return (int)(((kb + 1) * gridDim.x + total - 1) / total) - 1;
    }
    __device__ bool next(Item& it) {
        if (!stream) {
            if (w >= num_work) return false;
            it.tile = w % tiles;
            it.part = w / tiles;
            it.nparts = splits;
            it.kb0 = it.part * kb_per_split;
            it.nkb = min(kb_total, it.kb0 + kb_per_split) - it.kb0;
            w += stride;
            return true;
        }
        if (lo >= hi) return false;
        it.tile = (int)(lo / kb_total);
        it.kb0 = (int)(lo - (long long)it.tile * kb_total);
        it.nkb = (int)min((long long)(kb_total - it.kb0), hi - lo);
        lo += it.nkb;
        if (it.nkb == kb_total) { it.part = 0; it.nparts = 1; }
        else {
            const int first = owner((long long)it.tile * kb_total), last = owner((long long)(it.tile + 1) * kb_total - 1);
            it.part = (int)blockIdx.x - first;
            it.nparts = last - first + 1;
        }
        return true;
    }
};

template <int BN, bool ROPE>
__global__ void __launch_bounds__(THREADS, BN <= 16 ? GEMM_NARROW_CTAS : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, Epilogue ep, int kb_total, int kb_per_split, int tiles_a, int tiles_b, int num_work) {
    constexpr int STAGES = stages_for<BN>();
    constexpr int B_BYTES = BN * BK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    // two accumulators; a tile width that is no power of two takes the next one (TMEM is handed out in
    // powers of two)
    constexpr uint32_t ACC_COLS = BN <= 16 ? 16 : BN <= 32 ? 32 : BN <= 64 ? 64 : BN <= 128 ? 128 : 256;
    // Narrow tiles (few tokens): the four MMAs of a k-block go to four accumulators of their own, which
    // the epilogue adds up.  One accumulator would chain them, and an MMA of 16 columns is all latency:
    // measured 0.35 us per k-block and CTA, the same with the weights in L2 as in DRAM.
    constexpr uint32_t NSUB = BN <= 64 ? 4 : 1;
    constexpr uint32_t TMEM_COLS = 2 * NSUB * ACC_COLS < 32 ? 32 : 2 * NSUB * ACC_COLS;
    constexpr uint32_t IDESC = bw::umma_idesc_bf16(BM, BN);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    float* staging = (float*)(smem + STAGES * STAGE_BYTES);
    uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES + staging_bytes<BN>());
    // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);

    BW_PDL_TRIGGER();   // the next kernel in the stream may start launching
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = bw::smem_u32(bars), empty0 = bw::smem_u32(bars + STAGES);
    const uint32_t tfull0 = bw::smem_u32(bars + 2 * STAGES), tempty0 = bw::smem_u32(bars + 2 * STAGES + 2);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { bw::mbar_init(full0 + 8 * s, 1); bw::mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { bw::mbar_init(tfull0 + 8 * a, 1); bw::mbar_init(tempty0 + 8 * a, 4); }
        bw::fence_barrier_init();
        bw::tma_prefetch_desc(&tmA);
        bw::tma_prefetch_desc(&tmB);
        tmem_slot[1] = (uint32_t)g_status;   // an earlier timeout: later launches do no work
    }
    if (warp == 1) bw::tmem_alloc(bw::smem_u32(tmem_slot), TMEM_COLS);
    bw::tc_fence_before();
    __syncthreads();
    bw::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const bool dead = tmem_slot[1] != 0;
    const int tiles = tiles_a * tiles_b;

    if (dead) {
        // fall through to the exit
    } else if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            // In the transposed orientation A is the weight matrix, which no kernel writes: its tiles
            // for the first stages are requested before the wait for the earlier kernels, whose
            // results (the activations in B) are loaded after it.
            int ahead = 0;
            Items items(ep, kb_total, kb_per_split, tiles, num_work);
            Item im;
            if (ep.transposed) {
                Items peek = items;
                if (peek.next(im)) {
                    const int tile_a = im.tile % tiles_a;
                    ahead = min(im.nkb, STAGES);
                    for (int i = 0; i < ahead; ++i) {
                        bw::mbar_expect_tx(full0 + 8 * i, STAGE_BYTES);
                        bw::tma_load_2d(bw::smem_u32(smem + i * STAGE_BYTES), &tmA, full0 + 8 * i, (im.kb0 + i) * BK, tile_a * BM);
                    }
                }
            }
            BW_PDL_WAIT();
            while (ok && items.next(im)) {
                const int tile_a = im.tile % tiles_a, tile_b = im.tile / tiles_a;
                const int kb0 = im.kb0, nkb = im.nkb;
                for (int i = 0; i < nkb; ++i, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    const uint32_t a_dst = bw::smem_u32(smem + s * STAGE_BYTES);
                    if ((int)it < ahead) {   // A of this stage is already on its way
                        bw::tma_load_2d(a_dst + A_BYTES, &tmB, full0 + 8 * s, (kb0 + i) * BK, tile_b * BN);
                        continue;
                    }
                    if (!bw::mbar_wait(empty0 + 8 * s, ph ^ 1, &g_status, 1)) { ok = false; break; }
                    bw::mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                    bw::tma_load_2d(a_dst, &tmA, full0 + 8 * s, (kb0 + i) * BK, tile_a * BM);
                    bw::tma_load_2d(a_dst + A_BYTES, &tmB, full0 + 8 * s, (kb0 + i) * BK, tile_b * BN);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t it = 0, n = 0;
            bool ok = true;
            Items items(ep, kb_total, kb_per_split, tiles, num_work);
            Item im;
            for (; ok && items.next(im); ++n) {
                const int nkb = im.nkb;
                const uint32_t acc = n & 1, accph = (n >> 1) & 1;
                if (!bw::mbar_wait(tempty0 + 8 * acc, accph ^ 1, &g_status, 4)) break;   // epilogue drained it
                bw::tc_fence_after();
                const uint32_t tmem_acc = tmem_base + acc * NSUB * ACC_COLS;
                for (int i = 0; i < nkb; ++i, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!bw::mbar_wait(full0 + 8 * s, ph, &g_status, 2)) { ok = false; break; }
                    bw::tc_fence_after();
                    const uint32_t a_addr = bw::smem_u32(smem + s * STAGE_BYTES);
                    const uint64_t da = bw::umma_smem_desc_sw128(a_addr);
                    const uint64_t db = bw::umma_smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // advance 32 bytes (2 units of 16 B) along K inside the swizzle row
                        if constexpr (NSUB == 4) bw::umma_bf16(tmem_acc + k * ACC_COLS, da + 2 * k, db + 2 * k, IDESC, i != 0);
                        else bw::umma_bf16(tmem_acc, da + 2 * k, db + 2 * k, IDESC, (i | k) != 0);
                    }
                    bw::umma_commit(empty0 + 8 * s);   // the stage is free once these MMAs are done
                }
                bw::umma_commit(tfull0 + 8 * acc);     // this accumulator is complete
            }
        }
    } else {
        BW_PDL_WAIT();   // the outputs, the split-K scratch and its counters belong to earlier kernels until here
        const int quarter = warp & 3;              // TMEM lanes 32 * quarter .. + 31
        float* stage = staging + (warp - 2) * (32 * 33);
        const int a_rows = ep.transposed ? ep.features : ep.tokens;
        const int b_rows = ep.transposed ? ep.tokens : ep.features;
        const size_t plane = (size_t)ep.tokens * ep.features;
        constexpr int CH = BN < 32 ? 16 : 32;
        uint32_t n = 0;
        Items items(ep, kb_total, kb_per_split, tiles, num_work);
        Item im;
        for (; items.next(im); ++n) {
            const int tile = im.tile, split = im.part, nparts = im.nparts;
            const int tile_a = tile % tiles_a, tile_b = tile / tiles_a;
            const uint32_t acc = n & 1, accph = (n >> 1) & 1;
            if (!bw::mbar_wait(tfull0 + 8 * acc, accph, &g_status, 3)) break;
            bw::tc_fence_after();
            const uint32_t lane_addr = tmem_base + acc * NSUB * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
            const int ga = tile_a * BM + quarter * 32 + lane;   // this lane's row of A
            float* part = (ep.partial && nparts > 1) ? ep.partial + (size_t)split * plane : nullptr;
            int rope_kv = -1;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += CH) {
                uint32_t v[CH];
                if constexpr (CH == 32) bw::tmem_ld_32x32(lane_addr + c0, v);
                else bw::tmem_ld_32x16(lane_addr + c0, v);
                if constexpr (NSUB == 4) {   // (k-step 0 + 1) + (2 + 3), the same order everywhere
                    uint32_t v1[CH], v2[CH], v3[CH];
                    if constexpr (CH == 32) {
                        bw::tmem_ld_32x32(lane_addr + ACC_COLS + c0, v1); bw::tmem_ld_32x32(lane_addr + 2 * ACC_COLS + c0, v2);
                        bw::tmem_ld_32x32(lane_addr + 3 * ACC_COLS + c0, v3);
                    } else {
                        bw::tmem_ld_32x16(lane_addr + ACC_COLS + c0, v1); bw::tmem_ld_32x16(lane_addr + 2 * ACC_COLS + c0, v2);
                        bw::tmem_ld_32x16(lane_addr + 3 * ACC_COLS + c0, v3);
                    }
                    bw::tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < CH; ++c)
                        v[c] = __float_as_uint((__uint_as_float(v[c]) + __uint_as_float(v1[c])) +
                                               (__uint_as_float(v2[c]) + __uint_as_float(v3[c])));
                } else {
                    bw::tmem_ld_wait();
                }
                if (ep.transposed) {
                    // lanes hold 32 consecutive features, the columns are consecutive tokens: coalesced as it is
                    float vals[CH];
#pragma unroll
                    for (int c = 0; c < CH; ++c) vals[c] = __uint_as_float(v[c]);
                    const int token0 = tile_b * BN + c0;
                    emit<CH, ROPE>(ep, part, vals, token0, min(CH, b_rows - token0), ga, ga < a_rows);
                } else if (ep.tma_add) {
                    if constexpr (CH == 32 && !ROPE) {
                        // out += tile: the lane's row of 32 sums goes to a 128-byte-swizzled box in shared
                        // memory, the TMA unit adds the box into out (rows and columns past the matrix are
                        // clipped; columns past this tile's width are sent as zeros).  Two boxes per warp,
                        // so filling one overlaps the other's way out.
                        const int chunk = c0 / 32;
                        uint8_t* box = (uint8_t*)staging + ((warp - 2) * 2 + (chunk & 1)) * 4096;
                        if (lane == 0) bw::bulk_wait_group_read<1>();   // the box used two chunks ago has been read
                        __syncwarp();
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            uint4 q4;
                            q4.x = c0 + 4 * j + 0 < BN ? v[4 * j + 0] : 0u; q4.y = c0 + 4 * j + 1 < BN ? v[4 * j + 1] : 0u;
                            q4.z = c0 + 4 * j + 2 < BN ? v[4 * j + 2] : 0u; q4.w = c0 + 4 * j + 3 < BN ? v[4 * j + 3] : 0u;
                            *reinterpret_cast<uint4*>(box + lane * 128 + ((j ^ (lane & 7)) << 4)) = q4;
                        }
                        bw::fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            bw::tma_reduce_add_2d(&tmC, bw::smem_u32(box), tile_b * BN + c0, tile_a * BM + quarter * 32);
                            bw::bulk_commit_group();
                        }
                    }
                } else if (ep.swiglu && !part) {
                    if constexpr (CH == 32 && !ROPE) {
                        const int token = tile_a * BM + quarter * 32 + lane;
                        if (token < a_rows && tile_b * BN + c0 < b_rows) swiglu_direct(ep, v, token, tile_b * BN + c0);
                    }
                } else if (ROPE && !part) {
                    if constexpr (CH == 32 && ROPE) {
                        const int token = tile_a * BM + quarter * 32 + lane;
                        if (c0 == 0)   // once per tile: where this thread's token keeps its keys and values
                            rope_kv = (token < a_rows && ep.rope.kv_slot) ? __ldg(ep.rope.kv_slot + token) : -1;
                        if (token < a_rows && tile_b * BN + c0 < b_rows)
                            rope_direct(ep, v, token, tile_b * BN + c0, min(32, BN - c0), rope_kv);
                    }
                } else {
                    if constexpr (CH == 32) {
                        // turn the 32 x 32 block through shared memory so that a warp stores whole rows
#pragma unroll
                        for (int c = 0; c < 32; ++c) stage[lane * 33 + c] = __uint_as_float(v[c]);
                        __syncwarp();
                        const int feature = tile_b * BN + c0 + lane;
                        const int token0 = tile_a * BM + quarter * 32;
                        float vals[32];
#pragma unroll
                        for (int r = 0; r < 32; ++r) vals[r] = stage[r * 33 + lane];
                        __syncwarp();
                        if (tile_b * BN + c0 < b_rows)
                            emit<32, ROPE>(ep, part, vals, token0, min(32, a_rows - token0), feature,
                                           feature < b_rows && c0 + lane < BN);
                    }
                }
            }
            // the accumulator may be overwritten now
            bw::tc_fence_before();
            __syncwarp();
            if (lane == 0) bw::mbar_arrive(tempty0 + 8 * acc);

            if (part && ep.counters) {
                // split-K, reduced here: the warp that completes this (tile, quarter) last sums all
                // partials.  (Without counters a second kernel does the sums, in parallel: better for
                // many tokens.)  The warp's writes happen before lane 0's fence and counter update.
                __syncwarp();
                int last = 0;
                if (lane == 0) {
                    __threadfence();
                    last = atomicAdd(&ep.counters[tile * 4 + quarter], 1) == nparts - 1;
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    __threadfence();
                    // eight tokens at a time, so that their loads are in flight together
                    if (ep.transposed) {
                        const int t_end = min(b_rows, (tile_b + 1) * BN);
                        for (int token0 = tile_b * BN; token0 < t_end; token0 += 8) {
                            float vals[8];
#pragma unroll
                            for (int c = 0; c < 8; ++c) vals[c] = 0.f;
                            const int nv = min(8, t_end - token0);
                            RopeCtx<8> cx;
                            if constexpr (ROPE) rope_prefetch<8>(ep, cx, token0, nv, ga, ga < a_rows);
                            if (ga < a_rows)
                                for (int s0 = 0; s0 < nparts; s0 += 4) {   // four parts' loads in flight, added in part order
                                    float t[4][8];
#pragma unroll
                                    for (int j = 0; j < 4; ++j) {
                                        const float* src = ep.partial + (size_t)(s0 + j) * plane + (size_t)token0 * ep.features + ga;
#pragma unroll
                                        for (int c = 0; c < 8; ++c)
                                            t[j][c] = (s0 + j < nparts && c < nv) ? __ldcg(src + (size_t)c * ep.features) : 0.f;
                                    }
#pragma unroll
                                    for (int j = 0; j < 4; ++j)
                                        if (s0 + j < nparts) {
#pragma unroll
                                            for (int c = 0; c < 8; ++c) vals[c] += t[j][c];
                                        }
                                }
                            if constexpr (ROPE) rope_finish<8>(ep, cx, vals, token0, nv, ga < a_rows);
                            else emit<8, false>(ep, nullptr, vals, token0, nv, ga, ga < a_rows);
                        }
                    } else {
                        const int r_end = min(a_rows, tile_a * BM + quarter * 32 + 32);
                        for (int c0 = 0; c0 < BN && tile_b * BN + c0 < b_rows; c0 += 32) {
                            const int feature = tile_b * BN + c0 + lane;
                            for (int token0 = tile_a * BM + quarter * 32; token0 < r_end; token0 += 8) {
                                float vals[8];
#pragma unroll
                                for (int c = 0; c < 8; ++c) vals[c] = 0.f;
                                const int nv = min(8, r_end - token0);
                                if (feature < b_rows && c0 + lane < BN)
                                    for (int s = 0; s < nparts; ++s) {
                                        const float* src = ep.partial + (size_t)s * plane + (size_t)token0 * ep.features + feature;
#pragma unroll
                                        for (int c = 0; c < 8; ++c)
                                            if (c < nv) vals[c] += __ldcg(src + (size_t)c * ep.features);
                                    }
                                emit<8, ROPE>(ep, nullptr, vals, token0, nv, feature, feature < b_rows && c0 + lane < BN);
                            }
                        }
                    }
                    if (lane == 0) ep.counters[tile * 4 + quarter] = 0;
                }
            }
        }
    }
    if (ep.tma_add && warp >= 2 && lane == 0) bw::bulk_wait_group<0>();   // the boxes have left shared memory and landed
    bw::tc_fence_before();
    __syncthreads();
    if (warp == 1) bw::tmem_dealloc(tmem_base, TMEM_COLS);
}

// The same product for many tokens on CTA PAIRS (cta_group::2): a cluster of two CTAs takes a tile of
// 256 tokens x BN features.  Each CTA loads its 128 rows of x and HALF of the BN weight rows (so a
// k-block costs it 16 + BN / 8 KB instead of 16 + BN / 4: less traffic from L2 per flop, and room
// for more stages), the leader CTA's MMA thread issues one M = 256 instruction that reads both
// CTAs' shared memory and writes each CTA's 128 accumulator rows into its own TMEM, and each CTA
// runs the epilogue of its own rows.  Normal orientation only, no K split.
//   full[s]   on the leader: both CTAs' loads of stage s count their bytes there;
//   empty[s]  on each CTA: the leader's commit reaches both;
//   tfull[a]  on each CTA (the leader's commit reaches both); tempty[a] on the leader: the four
//             epilogue warps of BOTH CTAs arrive there.
template <int BN, bool ROPE>
__global__ void __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, Epilogue ep, int kb_total, int kb_per_split, int tiles_a, int tiles_b,
                 int num_work) {
    constexpr int BH = BN / 2;                       // weight rows this CTA loads
    constexpr int B_BYTES = BH * BK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int STAGES = pair_stages<BN>();
    constexpr uint32_t TMEM_COLS = 512;              // two accumulators of up to 256 columns
    constexpr uint32_t IDESC = bw::umma_idesc_bf16(2 * BM, BN);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    float* staging = (float*)(smem + STAGES * STAGE_BYTES);
    uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES + staging_bytes<BN>());
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);

    BW_PDL_TRIGGER();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = bw::cluster_ctarank();     // 0: the leader
    const uint32_t full0 = bw::smem_u32(bars), empty0 = bw::smem_u32(bars + STAGES);
    const uint32_t tfull0 = bw::smem_u32(bars + 2 * STAGES), tempty0 = bw::smem_u32(bars + 2 * STAGES + 2);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { bw::mbar_init(full0 + 8 * s, 1); bw::mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { bw::mbar_init(tfull0 + 8 * a, 1); bw::mbar_init(tempty0 + 8 * a, 8); }
        bw::fence_barrier_init();
        bw::tma_prefetch_desc(&tmA);
        bw::tma_prefetch_desc(&tmB);
        tmem_slot[1] = (uint32_t)g_status;
    }
    if (warp == 1) bw::tmem_alloc_pair(bw::smem_u32(tmem_slot), TMEM_COLS);
    bw::tc_fence_before();
    __syncthreads();
    bw::cluster_sync();                              // both CTAs' barriers exist before anyone arrives remotely
    bw::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const bool dead = tmem_slot[1] != 0;
    const int tiles = tiles_a * tiles_b;
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

    if (dead) {
        // fall through to the exit
    } else if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            Items items(ep, kb_total, kb_per_split, tiles, num_work, pair, n_pairs);
            Item im;
            BW_PDL_WAIT();
            while (ok && items.next(im)) {
                const int tile_a = im.tile % tiles_a, tile_b = im.tile / tiles_a;
                for (int i = 0; i < im.nkb; ++i, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!bw::mbar_wait(empty0 + 8 * s, ph ^ 1, &g_status, 31)) { ok = false; break; }
                    const uint32_t a_dst = bw::smem_u32(smem + s * STAGE_BYTES);
                    const uint32_t lead_full = bw::pair_leader_addr(full0 + 8 * s);
                    if (rank == 0) bw::mbar_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);   // the bytes of both CTAs
                    bw::tma_load_2d_pair(a_dst, &tmA, lead_full, (im.kb0 + i) * BK, tile_a * 2 * BM + (int)rank * BM);
                    bw::tma_load_2d_pair(a_dst + A_BYTES, &tmB, lead_full, (im.kb0 + i) * BK, tile_b * BN + (int)rank * BH);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            uint32_t it = 0, n = 0;
            bool ok = true;
            Items items(ep, kb_total, kb_per_split, tiles, num_work, pair, n_pairs);
            Item im;
            for (; ok && items.next(im); ++n) {
                const uint32_t acc = n & 1, accph = (n >> 1) & 1;
                if (!bw::mbar_wait_cluster(tempty0 + 8 * acc, accph ^ 1, &g_status, 34)) break;   // both epilogues drained it
                bw::tc_fence_after();
                const uint32_t tmem_acc = tmem_base + acc * 256;
                for (int i = 0; i < im.nkb; ++i, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!bw::mbar_wait_cluster(full0 + 8 * s, ph, &g_status, 32)) { ok = false; break; }
                    bw::tc_fence_after();
                    const uint32_t a_addr = bw::smem_u32(smem + s * STAGE_BYTES);
                    const uint64_t da = bw::umma_smem_desc_sw128(a_addr);
                    const uint64_t db = bw::umma_smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        bw::umma_bf16_pair(tmem_acc, da + 2 * k, db + 2 * k, IDESC, (i | k) != 0);
                    bw::umma_commit_pair(empty0 + 8 * s, 3);   // the stage is free in both CTAs
                }
                bw::umma_commit_pair(tfull0 + 8 * acc, 3);     // both CTAs' rows of the accumulator are complete
            }
        }
    } else {
        BW_PDL_WAIT();
        const int quarter = warp & 3;
        float* stage = staging + (warp - 2) * (32 * 33);
        const int a_rows = ep.tokens, b_rows = ep.features;
        uint32_t n = 0;
        Items items(ep, kb_total, kb_per_split, tiles, num_work, pair, n_pairs);
        Item im;
        for (; items.next(im); ++n) {
            const int tile_a = im.tile % tiles_a, tile_b = im.tile / tiles_a;
            const uint32_t acc = n & 1, accph = (n >> 1) & 1;
            if (!bw::mbar_wait_cluster(tfull0 + 8 * acc, accph, &g_status, 33)) break;
            bw::tc_fence_after();
            const uint32_t lane_addr = tmem_base + acc * 256 + ((uint32_t)(quarter * 32) << 16);
            const int row0 = tile_a * 2 * BM + (int)rank * BM + quarter * 32;   // first token of this warp
            float* part = (ep.partial && im.nparts > 1) ? ep.partial + (size_t)im.part * ((size_t)ep.tokens * ep.features) : nullptr;
            int rope_kv = -1;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t v[32];
                bw::tmem_ld_32x32(lane_addr + c0, v);
                bw::tmem_ld_wait();
                if (part) {
                    // a K split: this item's sums go to its plane of the scratch as they are (the lane's token,
                    // 32 consecutive features); a second kernel adds the planes in split order
                    const int token = row0 + lane, f0 = tile_b * BN + c0;
                    if (token < a_rows && c0 < BN) {
                        float* dst = part + (size_t)token * ep.features + f0;
                        if ((ep.features & 3) == 0 && f0 + 32 <= b_rows) {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                *reinterpret_cast<uint4*>(dst + 4 * j) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                        } else {
#pragma unroll
                            for (int c = 0; c < 32; ++c)
                                if (f0 + c < b_rows && c0 + c < BN) dst[c] = __uint_as_float(v[c]);
                        }
                    }
                } else if (ep.tma_add) {
                    if constexpr (!ROPE) {
                        const int chunk = c0 / 32;
                        uint8_t* box = (uint8_t*)staging + ((warp - 2) * 2 + (chunk & 1)) * 4096;
                        if (lane == 0) bw::bulk_wait_group_read<1>();
                        __syncwarp();
#pragma unroll
                        for (int j = 0; j < 8; ++j) {   // columns past this tile's width go out as zeros
                            const bool in = c0 + 4 * j < BN;   // BN is a multiple of 16: whole groups of four
                            *reinterpret_cast<uint4*>(box + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                                in ? make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]) : make_uint4(0u, 0u, 0u, 0u);
                        }
                        bw::fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            bw::tma_reduce_add_2d(&tmC, bw::smem_u32(box), tile_b * BN + c0, row0);
                            bw::bulk_commit_group();
                        }
                    }
                } else if (ROPE) {
                    if constexpr (ROPE) {
                        const int token = row0 + lane;
                        if (c0 == 0) rope_kv = (token < a_rows && ep.rope.kv_slot) ? __ldg(ep.rope.kv_slot + token) : -1;
                        if (token < a_rows && tile_b * BN + c0 < b_rows)
                            rope_direct(ep, v, token, tile_b * BN + c0, min(32, BN - c0), rope_kv);
                    }
                } else if (ep.swiglu) {
                    if (row0 + lane < a_rows && tile_b * BN + c0 < b_rows) swiglu_direct(ep, v, row0 + lane, tile_b * BN + c0);
                } else {
#pragma unroll
                    for (int c = 0; c < 32; ++c) stage[lane * 33 + c] = __uint_as_float(v[c]);
                    __syncwarp();
                    const int feature = tile_b * BN + c0 + lane;
                    float vals[32];
#pragma unroll
                    for (int r = 0; r < 32; ++r) vals[r] = stage[r * 33 + lane];
                    __syncwarp();
                    if (tile_b * BN + c0 < b_rows)
                        emit<32, false>(ep, nullptr, vals, row0, min(32, a_rows - row0), feature,
                                        feature < b_rows && c0 + lane < BN);
                }
            }
            bw::tc_fence_before();
            __syncwarp();
            if (lane == 0) bw::mbar_arrive_cluster(bw::pair_leader_addr(tempty0 + 8 * acc));
        }
        if (ep.tma_add && lane == 0) bw::bulk_wait_group<0>();
    }
    bw::tc_fence_before();
    __syncthreads();
    bw::cluster_sync();   // nobody leaves while the other CTA may still arrive on its barriers or read its tiles
    if (warp == 1) bw::tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

// Split-K with many tokens: out = epilogue(sum over splits of partial), one thread per (token,
// feature), splits added in order.  SwiGLU: one thread per (token, output feature) reads its gate
// and up sums from the interleaved layout.
__global__ void splitk_reduce_kernel(Epilogue ep) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    const size_t plane = (size_t)ep.tokens * ep.features;
    const int width = ep.swiglu ? ep.features / 2 : ep.features;
    const size_t total = (size_t)ep.tokens * width;
    if (!ep.swiglu && !ep.rope_on && ep.out_type == BW_F32 && (ep.features & 3) == 0 && (ep.ldo & 3) == 0 &&
        ((uintptr_t)ep.out & 15) == 0) {
        // float32 result, four features a thread: 16-byte loads of every plane, one 16-byte store
        const size_t quads = total / 4;
        for (size_t q = (size_t)blockIdx.x * blockDim.x + threadIdx.x; q < quads; q += (size_t)gridDim.x * blockDim.x) {
            const size_t i = q * 4;
            const int token = (int)(i / ep.features), j = (int)(i - (size_t)token * ep.features);
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < ep.splits; ++s) {
                const float4 t = *reinterpret_cast<const float4*>(ep.partial + (size_t)s * plane + i);
                v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w;
            }
            if (ep.bias) { v.x += bias_at(ep, j); v.y += bias_at(ep, j + 1); v.z += bias_at(ep, j + 2); v.w += bias_at(ep, j + 3); }
            float4* o = reinterpret_cast<float4*>((float*)ep.out + (size_t)token * ep.ldo + j);
            if (ep.accumulate) { const float4 old = *o; v.x = old.x + v.x; v.y = old.y + v.y; v.z = old.z + v.z; v.w = old.w + v.w; }
            *o = v;
        }
        return;
    }
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int token = (int)(i / width), j = (int)(i - (size_t)token * width);
        if (ep.swiglu) {
            const int fg = (j / SWIGLU_BLOCK) * 2 * SWIGLU_BLOCK + j % SWIGLU_BLOCK, fu = fg + SWIGLU_BLOCK;
            float g = 0.f, u = 0.f;
            for (int s = 0; s < ep.splits; ++s) {
                g += ep.partial[(size_t)s * plane + (size_t)token * ep.features + fg];
                u += ep.partial[(size_t)s * plane + (size_t)token * ep.features + fu];
            }
            ((bf16*)ep.out)[(size_t)token * ep.ldo + j] = __float2bfloat16_rn(__fdividef(g, 1.f + __expf(-g)) * u);
            continue;
        }
        if (ep.rope_on) {
            const RopeSlot sl = rope_slot(ep.rope, j);
            float x = 0.f, partner = 0.f;
            for (int s = 0; s < ep.splits; ++s) {
                x += ep.partial[(size_t)s * plane + i];
                if (sl.rot) partner += ep.partial[(size_t)s * plane + (i ^ 1)];
            }
            const int kvh = sl.head < ep.rope.nh + ep.rope.nkv ? sl.head - ep.rope.nh : sl.head - ep.rope.nh - ep.rope.nkv;
            const long long row = (sl.head >= ep.rope.nh && ep.rope.kv_slot) ? rope_page_row(ep.rope, __ldg(ep.rope.kv_slot + token), kvh) : -1;
            rope_store(ep.rope, sl, token, row, rope_angle(ep.rope, sl, token), x + bias_at(ep, j), partner + bias_at(ep, j ^ 1));
            continue;
        }
        float v = 0.f;
        for (int s = 0; s < ep.splits; ++s) v += ep.partial[(size_t)s * plane + i];
        if (ep.bias) v += ep.bias_type == BW_F32 ? ((const float*)ep.bias)[j] : __bfloat162float(((const bf16*)ep.bias)[j]);
        const size_t off = (size_t)token * ep.ldo + j;
        if (ep.out_type == BW_F32) {
            float* o = (float*)ep.out + off;
            *o = ep.accumulate ? *o + v : v;
        } else {
            ((bf16*)ep.out)[off] = __float2bfloat16_rn(v);
        }
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

template <int BN, bool ROPE>
int launch(const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& c, const Epilogue& ep, int kb_total, int kb_per_split,
           int tiles_a, int tiles_b, int num_work, cudaStream_t s) {
    constexpr int STAGES = stages_for<BN>();
    constexpr int smem = STAGES * (A_BYTES + BN * BK * 2) + staging_bytes<BN>() + (2 * STAGES + 4) * 8 + 16 + 1024;
    static_assert(smem <= 227 * 1024, "shared memory budget");
    static bool attr_done[bw::MAX_DEVICES];
    if (cudaError_t e = bw::allow_dynamic_smem(gemm_tc_kernel<BN, ROPE>, smem, attr_done); e != cudaSuccess) return (int)e;
    const int NUM_SMS = bw::num_sms();
    const int grid = num_work < NUM_SMS ? num_work : NUM_SMS;
    bw::launch((gemm_tc_kernel<BN, ROPE>), dim3(grid), dim3(THREADS), smem, s, a, b, c, ep, kb_total, kb_per_split,
               tiles_a, tiles_b, num_work);
    BW_LAUNCH_CHECK();
    return 0;
}

template <int BN, bool ROPE>
int launch_pair(const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& c, const Epilogue& ep, int kb_total,
                int kb_per_split, int tiles_a, int tiles_b, cudaStream_t s) {
    constexpr int STAGES = pair_stages<BN>();
    constexpr int smem = STAGES * (A_BYTES + (BN / 2) * BK * 2) + staging_bytes<BN>() + (2 * STAGES + 4) * 8 + 16 + 1024;
    static_assert(smem <= 227 * 1024, "shared memory budget");
    static bool attr_done[bw::MAX_DEVICES];
    if (cudaError_t e = bw::allow_dynamic_smem(gemm_pair_kernel<BN, ROPE>, smem, attr_done); e != cudaSuccess) return (int)e;
    const int NUM_SMS = bw::num_sms();
    const int num_work = tiles_a * tiles_b * (ep.splits > 1 ? ep.splits : 1);
    const int pairs = num_work < NUM_SMS / 2 ? num_work : NUM_SMS / 2;
    bw::launch_pairs((gemm_pair_kernel<BN, ROPE>), dim3(2 * pairs), dim3(THREADS), smem, s, a, b, c, ep, kb_total, kb_per_split,
                     tiles_a, tiles_b, num_work);
    BW_LAUNCH_CHECK();
    return 0;
}

// float32 [rows, cols] with row stride ld (elements), box = 32 x 32, 128-byte swizzle: the epilogue's
// way out for out += product
bool make_out_map(CUtensorMap* m, void* base, long long rows, long long cols, long long ld) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
    cuuint32_t box[2] = {32, 32};
    cuuint32_t estr[2] = {1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

}  // namespace

// The number of SMs the planners and launchers count with (the current device's; 148 where none can be asked).
BW_EXPORT int bw_num_sms() { return bw::num_sms(); }

// Whether bw_gemm_tc takes these operands: bf16, K a multiple of 8 (a TMA row stride
// is a multiple of 16 bytes), 16-byte aligned bases and strides.
BW_EXPORT int bw_gemm_tc_supported(const void* x, const void* w, int K, long long ldx) {
    return (K > 0 && K % 8 == 0 && ldx % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0) ? 1 : 0;
}

// Picks the orientation, the tile width and the number of K splits for
// out[M, N] = x[M, K] . w[N, K]^T.  Returns splits; *transposed and *bn are set.
BW_EXPORT int bw_gemm_tc_plan(int M, int N, int K, int swiglu, long long workspace_elems, long long n_counters,
                              int* transposed, int* bn) {
    const int NUM_SMS = bw::num_sms();
    const int kb_total = ceil_div(K, BK);
    int tr = M <= 256, b;
    if (tr) { b = 16; while (b < M) b *= 2; }
    else {
        // The width of the tile (a multiple of 16; of 32 for SwiGLU, whose epilogue works on 16 gate
        // and 16 up features at a time) is the one whose rounds over the 148 persistent CTAs cost
        // least: a round costs its width, a 128-wide tile 10 % more per column (both operands then
        // stream from shared memory at the same rate as the MMA consumes them).
        const int widths[4] = {256, 240, 224, 128};   // (176 was measured: slower per column than it saves)
        double best_cost = 0.0; b = 256;
        for (int i = 0; i < 4; ++i) {
            const int wd = widths[i];
            if (swiglu && wd % 32) continue;
            const long long t = (long long)ceil_div(M, BM) * ceil_div(N, wd);
            const double cost = (double)ceil_div(t, NUM_SMS) * wd * (wd == 128 ? 1.0 / 0.9 : 1.0);
            if (i == 0 || cost < best_cost * 0.995) { best_cost = cost; b = wd; }
        }
    }
    *transposed = tr; *bn = b;
    const long long tiles = tr ? (long long)ceil_div(N, BM) * ceil_div(M, b) : (long long)ceil_div(M, BM) * ceil_div(N, b);
    // Timings of the decode shapes on a B200 (back-to-back launches in a CUDA graph, cold weights)
    // say: with at least one tile per SM do not split; with fewer, split so that one round of
    // items just fills the SMs, keeping 8 or more k-blocks per item, and the float32 partial
    // sums (2 * s * M * N * 4 bytes written and read) well below the weight bytes (N * K * 2).
    int best = 1;
    if (tiles < NUM_SMS) {
        best = (int)(NUM_SMS / tiles);
        if (best > kb_total / 8) best = kb_total / 8;
        if (M > 64 && best > K / (8 * M)) best = K / (8 * M);
        if (best > 16) best = 16;
        while (best > 1 && ((long long)best * M * N > workspace_elems || tiles * 4 > n_counters)) --best;
        if (best < 1) best = 1;
    }
    return best;
}

// The estimates below count time in units of one feature column times one k-block on a tile of 256 tokens
// at the rate of a CTA pair (1.7 ns).  Adding the planes of a K split costs a second kernel (2.5 us) and
// (splits + 2) passes over the float32 result at about 5 TB/s (the planes mostly stay in L2).
namespace {
double split_sum_cost(int M, int N, int s) {
    return s <= 1 ? 0.0 : (2.5e-6 + (double)(s + 2) * M * N * 4.0 / 5e12) / 1.73e-9;
}
// single CTAs on tiles of 128 tokens x bn features: measured 15-20 % slower per flop than pairs at 224 to 256
// columns, and at 53-66 % of a pair's rate at 128 columns (steps of 512 tokens, o and down of the 8B shape)
double gemm_single_cost(int M, int N, int K, int bn, long long tiles, int splits) {
    const int NUM_SMS = bw::num_sms();
    const int kb_total = ceil_div(K, BK);
    return (double)ceil_div(tiles * splits, NUM_SMS) * ceil_div(kb_total, splits) * bn * (bn == 128 ? 1.7 : 1.18) +
           split_sum_cost(M, N, splits);
}
}  // namespace

// CTA pairs for out[M, N] = x[M, K] . w[N, K]^T with M > 256: the tile width (256 or 224) and the number of K
// splits (1 to 4, each of 8 k-blocks or more, their planes within the scratch) with the lowest estimate, which
// is returned (negative: pairs cannot take it).  force_splits > 0 fixes the splits.
BW_EXPORT double bw_gemm_tc_pair_plan(int M, int N, int K, int force_splits, long long workspace_elems, int* width, int* splits) {
    const int NUM_SMS = bw::num_sms();
    const int kb_total = ceil_div(K, BK), pa = ceil_div(M, 2 * BM);
    const int widths[2] = {256, 224};   // (240 works but was measured no faster than 256)
    double best = -1.0;
    for (int i = 0; i < 2; ++i) {
        const long long t = (long long)pa * ceil_div(N, widths[i]);
        for (int ps = 1; ps <= 4; ++ps) {
            if (force_splits > 0 && ps != (force_splits > kb_total ? kb_total : force_splits)) continue;
            // Measured on the 8B layer sizes at 300 to 1,024 tokens: a split pays only as TWO halves of a long K
            // (128 k-blocks or more: the down projection) whose items still fit one round of the 74 pairs
            // (down at 300 tokens: 59 against 73 us; at 512: 68 against 72); everywhere else the planes'
            // way through memory costs more than the idle pairs (o at 512 tokens: 38 against 26 us).
            if (ps > 1 && force_splits <= 0 && (ps != 2 || kb_total < 128 || t * ps > NUM_SMS / 2)) continue;
            if (ps > kb_total || (ps > 1 && (long long)ps * M * N > workspace_elems)) continue;
            const double cost = (double)ceil_div(t * ps, NUM_SMS / 2) * ceil_div(kb_total, ps) * widths[i] + split_sum_cost(M, N, ps);
            if (best < 0.0 || cost < best * 0.995) { best = cost; *width = widths[i]; *splits = ps; }
        }
    }
    return best;
}

constexpr int PLANES_MAX_TOKENS = 256;   // bw_gemm_tc_planes: the orientation with the features in the 128-row dimension

// out[M, N] (=|+=) x[M, K] . w[N, K]^T (+ bias[N]).  x, w bf16; out float32 or bf16
// (accumulate: float32).  swiglu != 0: w holds gate and up rows interleaved in blocks of 16
// (16 gate rows, the 16 up rows of the same features, ...), N = 2 I with I a multiple of 16,
// and out is bf16 [M, I] = silu(gate) * up.  workspace / counters: scratch for split-K
// (float32 partial sums; int32 counters that are zero between launches); may be null.
// force_splits > 0 overrides the planner.
static int run_gemm_tc(const void* x, const void* w, const void* bias, int bias_type, void* out, int out_type,
                       int M, int N, int K, long long ldx, long long ldo, int accumulate, int swiglu,
                       float* workspace, long long workspace_elems, int* counters, long long n_counters,
                       int force_splits, const RopeOut* rope, void* stream, int* planes_out = nullptr) {
    if (M <= 0 || N <= 0) return 0;
    // planes_out: the product is left as *planes_out float32 planes [M, N] in `out` (row stride N, the bias
    // in the first), to be added up by its reader; K is split as if the sums were made here.
    const bool planes = planes_out != nullptr;
    if (planes && (M > PLANES_MAX_TOKENS || out_type != BW_F32 || accumulate || swiglu || rope || ldo != N ||
                   workspace != (float*)out))
        return BW_ERR_BAD_ARG;
    const int NUM_SMS = bw::num_sms();
    if (!bw_gemm_tc_supported(x, w, K, ldx)) return BW_ERR_UNSUPPORTED;
    if (accumulate && out_type != BW_F32) return BW_ERR_BAD_ARG;
    if (swiglu && (N % (2 * SWIGLU_BLOCK) != 0 || out_type != BW_BF16 || accumulate || bias || ldo < N / 2))
        return BW_ERR_BAD_ARG;
    if (rope && (swiglu || accumulate)) return BW_ERR_BAD_ARG;
    if (!swiglu && !rope && ldo < N) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const bool can_split = workspace && (counters || planes);
    if (planes) n_counters = 1LL << 40;   // no counters are used: nothing to run out of
    int tr, bn;
    int splits = bw_gemm_tc_plan(M, N, K, swiglu, can_split ? workspace_elems : 0, can_split ? n_counters : 0, &tr, &bn);
    if (!tr && bn < 128) return BW_ERR_BAD_ARG;   // only tiles of 128 columns or more have the normal orientation's staging
    const int kb_total = ceil_div(K, BK);
    const long long a_rows = tr ? N : M, b_rows = tr ? M : N;
    const int tiles_a = ceil_div(a_rows, BM), tiles_b = ceil_div(b_rows, bn);
    if (force_splits > 0) {
        splits = force_splits > kb_total ? kb_total : force_splits;
        if (splits > 1 && (!can_split || (long long)splits * M * N > workspace_elems ||
                           (long long)tiles_a * tiles_b * 4 > n_counters))
            return BW_ERR_BAD_ARG;
    }
    // More than 256 tokens: CTA pairs on tiles of 256 tokens, or single CTAs: whichever the estimate says
    // is faster (mode 0: never pairs; 1: the estimate; 2: pairs whenever they can; BW_GEMM_PAIR or
    // bw_gemm_tc_pair_mode).  With few tiles for the 74 pairs (steps of 300 to 1,000 tokens on the
    // products with few output features) the pairs split K as well; the partial sums are added in split
    // order by the second kernel.
    if (g_pair_mode < 0) { const char* e = getenv("BW_GEMM_PAIR"); g_pair_mode = (e && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 1; }
    int pbn = 256, psplits = 1;
    bool use_pairs = false;
    if (g_pair_mode > 0 && !tr && M > 256) {
        const double pair = bw_gemm_tc_pair_plan(M, N, K, force_splits, can_split ? workspace_elems : 0, &pbn, &psplits);
        const double single = gemm_single_cost(M, N, K, bn, (long long)tiles_a * tiles_b, splits);
        use_pairs = pair >= 0.0 && (g_pair_mode == 2 || pair <= single);
        if (use_pairs) splits = psplits;
    }
    const int kb_per_split = ceil_div(kb_total, splits);
    splits = ceil_div(kb_total, kb_per_split);   // no empty split

    CUtensorMap ta, tb;
    const void* a_ptr = tr ? w : x; const void* b_ptr = tr ? x : w;
    const long long a_ld = tr ? K : ldx, b_ld = tr ? ldx : K;
    if (!make_map(&ta, a_ptr, a_rows, K, a_ld, BM) || !make_map(&tb, b_ptr, b_rows, K, b_ld, bn)) return BW_ERR_DRIVER;

    Epilogue ep;
    // few tokens: the last warp of each tile sums the splits inside the kernel; more: a second kernel
    const bool fused_reduce = M <= FUSED_REDUCE_MAX_TOKENS;
    // Few tokens and more tiles than SMs, not a multiple of them (gate/up, the head): whole tiles leave
    // the last round partly empty, and the SMs that still work cannot draw the whole bandwidth (a CTA
    // of this kernel streams about 40 GB/s).  The k-blocks are dealt out in equal ranges instead:
    // gate/up at batch 8 takes 43 us instead of 47.5.  (Two CTAs per SM on whole tiles took 38 us when
    // the block scheduler spread them and 48 us when it paired them on some SMs and left others idle.)
    const long long n_tiles = (long long)tiles_a * tiles_b;
    const bool stream_k = tr && fused_reduce && can_split && !planes && force_splits <= 0 && splits == 1 && n_tiles > NUM_SMS &&
                          n_tiles % NUM_SMS != 0 && 2LL * M * N <= workspace_elems && n_tiles * 4 <= n_counters;
    if (stream_k) splits = 2;   // at most two CTAs share a tile: two planes of partial sums
    ep.out = out; ep.partial = splits > 1 ? workspace : nullptr; ep.counters = (fused_reduce && !planes) ? counters : nullptr;
    ep.planes = planes ? 1 : 0;
    if (planes) *planes_out = splits;
    ep.bias = bias; ep.ldo = ldo;
    ep.out_type = out_type; ep.bias_type = bias_type; ep.accumulate = accumulate; ep.transposed = tr;
    ep.swiglu = swiglu; ep.tokens = M; ep.features = N; ep.splits = splits;
    ep.rope_on = rope ? 1 : 0;
    ep.stream = stream_k ? 1 : 0;
    if (rope) ep.rope = *rope; else ep.rope = RopeOut{};
    // out += product with many tokens and no split: the epilogue hands 32 x 32 boxes to the TMA unit
    CUtensorMap tc;
    std::memset(&tc, 0, sizeof(tc));
    ep.tma_add = 0;
    if (!tr && accumulate && !bias && splits == 1 && !rope && !swiglu && ((uintptr_t)out & 15) == 0 && ldo % 4 == 0) {
        if (!make_out_map(&tc, out, M, N, ldo)) return BW_ERR_DRIVER;
        ep.tma_add = 1;
    }
    const int num_work = stream_k ? NUM_SMS : tiles_a * tiles_b * splits;
    int rc;
#define BW_GEMM_LAUNCH(R) switch (bn) { \
        case 16: rc = launch<16, R>(ta, tb, tc, ep, kb_total, kb_per_split, tiles_a, tiles_b, num_work, s); break; \
        case 32: rc = launch<32, R>(ta, tb, tc, ep, kb_total, kb_per_split, tiles_a, tiles_b, num_work, s); break; \
        case 64: rc = launch<64, R>(ta, tb, tc, ep, kb_total, kb_per_split, tiles_a, tiles_b, num_work, s); break; \
        case 128: rc = launch<128, R>(ta, tb, tc, ep, kb_total, kb_per_split, tiles_a, tiles_b, num_work, s); break; \
        case 224: rc = launch<224, R>(ta, tb, tc, ep, kb_total, kb_per_split, tiles_a, tiles_b, num_work, s); break; \
        case 240: rc = launch<240, R>(ta, tb, tc, ep, kb_total, kb_per_split, tiles_a, tiles_b, num_work, s); break; \
        case 256: rc = launch<256, R>(ta, tb, tc, ep, kb_total, kb_per_split, tiles_a, tiles_b, num_work, s); break; \
        default: return BW_ERR_BAD_ARG; }
    if (use_pairs) {
        CUtensorMap tb2;
        if (!make_map(&tb2, b_ptr, b_rows, K, b_ld, pbn / 2)) return BW_ERR_DRIVER;
        const int pa = ceil_div(M, 2 * BM), pb = ceil_div(N, pbn);
#define BW_PAIR_LAUNCH(W) (rope ? launch_pair<W, true>(ta, tb2, tc, ep, kb_total, kb_per_split, pa, pb, s) \
                                : launch_pair<W, false>(ta, tb2, tc, ep, kb_total, kb_per_split, pa, pb, s))
        rc = pbn == 256 ? BW_PAIR_LAUNCH(256) : BW_PAIR_LAUNCH(224);
#undef BW_PAIR_LAUNCH
    } else
    if (rope) BW_GEMM_LAUNCH(true) else BW_GEMM_LAUNCH(false)
#undef BW_GEMM_LAUNCH
    if (rc) return rc;
    if (splits > 1 && !fused_reduce && !planes) {
        const size_t total = (size_t)M * (swiglu ? N / 2 : N);
        const size_t want = (total + 255) / 256;
        const int blocks = (int)(want < (size_t)NUM_SMS * 8 ? want : (size_t)NUM_SMS * 8);
        bw::launch((splitk_reduce_kernel), dim3(blocks), dim3(256), 0, s, ep);
        BW_LAUNCH_CHECK();
    }
    return 0;
}

BW_EXPORT int bw_gemm_tc(const void* x, const void* w, const void* bias, int bias_type, void* out, int out_type,
                         int M, int N, int K, long long ldx, long long ldo, int accumulate, int swiglu,
                         float* workspace, long long workspace_elems, int* counters, long long n_counters,
                         int force_splits, void* stream) {
    return run_gemm_tc(x, w, bias, bias_type, out, out_type, M, N, K, ldx, ldo, accumulate, swiglu, workspace,
                       workspace_elems, counters, n_counters, force_splits, nullptr, stream);
}

// The product of up to 256 tokens as float32 planes: planes[p][m][n] for p < *n_planes add up to
// x[M, K] . w[N, K]^T (+ bias, which is part of plane 0), in plane order.  K is split as bw_gemm_tc
// would split it, but no CTA waits for another's partial sums: the kernel that reads the result adds
// the planes (bw_add_rmsnorm, bw_add_planes, bw_rope_append).  planes_elems: room in `planes` (floats).
BW_EXPORT int bw_gemm_tc_planes(const void* x, const void* w, const void* bias, int bias_type, float* planes,
                                long long planes_elems, int M, int N, int K, long long ldx, int force_splits,
                                int* n_planes, void* stream) {
    if (!planes || !n_planes || planes_elems < (long long)M * N) return BW_ERR_BAD_ARG;
    *n_planes = 1;
    return run_gemm_tc(x, w, bias, bias_type, planes, BW_F32, M, N, K, ldx, N, 0, 0, planes, planes_elems, nullptr, 0,
                       force_splits, nullptr, stream, n_planes);
}

// The fused q/k/v projection with rotary position encoding: x[M, K] . w[N, K]^T (+ bias), N =
// (nh + 2 nkv) * hd, the rows of w (and bias) of every q and k head ordered so that rows 2j and
// 2j + 1 are channels j and j + rd / 2 (rows from rd on, and the v heads, in place).  Rotated
// queries go to q_out [M, nh * hd] (bf16), rotated keys and raw values (bf16) to the pages
// [num_pages, nkv, page_size, hd] at kv_slot[token] = page * page_size + slot (-1: nowhere; a null
// kv_slot writes no keys or values).  table: float32 [M, rd], cosines then sines of every
// token's angles.
BW_EXPORT int bw_gemm_tc_rope(const void* x, const void* w, const void* bias, int bias_type, int M, int K,
                              long long ldx, const float* table, const int* kv_slot, void* q_out, void* k_pages,
                              void* v_pages, int nh, int nkv, int hd, int rd, int page_size,
                              float* workspace, long long workspace_elems, int* counters, long long n_counters,
                              int force_splits, void* stream) {
    if (nh <= 0 || nkv <= 0 || hd <= 0 || hd % 2 || rd < 0 || rd % 2 || rd > hd || page_size <= 0 || (rd > 0 && !table))
        return BW_ERR_BAD_ARG;
    RopeOut ro;
    ro.table = table; ro.kv_slot = kv_slot;
    ro.q_out = (bf16*)q_out; ro.k_pages = (bf16*)k_pages; ro.v_pages = (bf16*)v_pages;
    ro.nh = nh; ro.nkv = nkv; ro.hd = hd; ro.rd = rd; ro.page_size = page_size;
    return run_gemm_tc(x, w, bias, bias_type, nullptr, BW_BF16, M, (nh + 2 * nkv) * hd, K, ldx, 0, 0, 0, workspace,
                       workspace_elems, counters, n_counters, force_splits, &ro, stream);
}

// When products of more than 256 tokens run on CTA pairs: 0 never, 1 when the estimate says they are
// faster (the default), 2 whenever the product allows it (tests).  Returns the mode before.
BW_EXPORT int bw_gemm_tc_pair_mode(int mode) {
    const int old = g_pair_mode;
    if (mode >= 0 && mode <= 2) g_pair_mode = mode;
    return old;
}

// Reads and clears the status word (synchronises the device).  0: no wait ever gave up.
BW_EXPORT int bw_gemm_tc_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
    return v;
}
