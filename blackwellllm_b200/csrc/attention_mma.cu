// Paged causal grouped-query flash attention for bfloat16, head size HEAD_DIM (a
// compile-time multiple of 16, at most 256; the library is built per head size).
// Tensor-core products with mma.sync m16n8k16 (bf16 in, fp32 out); scores, the
// running maximum, the running sum and the output accumulator are float32; the
// probabilities are rounded to bfloat16 for the P.V product.
//
// The query heads of one kv head are stacked into the row dimension: row = token *
// G + head-in-group.  Two kernels share the same inner loop over 64-key tiles that
// cp.async gathers page by page into padded shared memory (double buffered):
//   * attn_rows_kernel: a work item is 64 rows of one (request, kv head); each of
//     the 4 warps owns 16 rows and walks all keys up to the causal diagonal.
//     For prompt portions (more than 16 rows).
//   * attn_keys_kernel: a work item is all (at most 16) rows of one (request, kv
//     head) over one slice of the keys; the 4 warps split each tile's keys and are
//     merged at the end; slices are merged by attn_merge_kernel.  For decode tokens.
// Keys beyond the request's length and pages the block table no longer holds are
// zero-filled in shared memory and masked, so stale cache contents never matter.
#include "tcgen05.cuh"   // mbarrier and TMA helpers (and common.cuh)

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<multiple of 16>"
#endif

using bf16 = __nv_bfloat16;

namespace {

constexpr int HD = HEAD_DIM;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size must be a multiple of 16 in [16, 256]");
constexpr int BN = 64;                 // keys per tile
constexpr int NWARPS = 4;
constexpr int THREADS = NWARPS * 32;
constexpr int ROW_BYTES = HD * 2 + 16; // padded row: ldmatrix rows land in distinct 16-byte bank groups
constexpr int KSTEPS = HD / 16;
constexpr int CPR = HD / 8;            // 16-byte chunks per row
constexpr int TILE_BYTES = BN * ROW_BYTES;
constexpr int SMEM_KEYS_MERGE_BYTES = (2 * NWARPS * 16 + NWARPS * 16 * HD) * 4;   // finish_keys

struct Params {
    const bf16* q; const bf16* k_pages; const bf16* v_pages; bf16* out;
    const int* cu_q; const int* q_start; const int* kv_len; const int* block_table;
    const int* work;              // int4 per item
    float* part_o; float* part_ml; // slices' partial results (attn_keys_kernel)
    int max_blocks, nh, nkv, G, page_size, num_pages, window;
    float scale_log2;
    // Decode rows straight from the q/k/v product (attn_keys_tma_kernel only; null: q holds the queries and
    // the cache this step's keys and values): qkv is float32 [planes][tokens][(nh + 2 nkv) * HD] to be added
    // up in plane order, the rotated channels of the q and k heads as (channel j, channel j + rd / 2) pairs;
    // rope_table is [tokens][rd] (cosines, then sines); append != 0: the CTA whose slice holds the token's
    // own position writes the rotated key and the value to the cache.  Every request has one token.
    const float* qkv; long long qkv_plane_stride; const float* rope_table;
    int qkv_planes, rd, append;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;  // 0: nothing is read, 16 zero bytes are written
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// barrier among the 128 compute threads only (a TMA producer warp, where there is one, stays out)
__device__ __forceinline__ void sync_compute_warps() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Gathers keys [key0, key0 + BN) of kv head g into a K and a V tile (padded rows).
__device__ __forceinline__ void load_kv_tile(const Params& p, const int* bt, int g, int kv_len, int key0,
                                             uint8_t* k_tile, uint8_t* v_tile) {
    if constexpr (THREADS % CPR == 0) {
        // each thread owns one 16-byte column and every (THREADS / CPR)-th row: the block index and
        // the slot in the page advance by additions, the page id is looked up once per page
        constexpr int RPP = THREADS / CPR;
        const int ch = threadIdx.x % CPR;
        int row = threadIdx.x / CPR;
        int kp = key0 + row;
        int blk = kp / p.page_size, slot = kp - blk * p.page_size;
        int cur_blk = -1, page = -1;
#pragma unroll 4
        for (; row < BN; row += RPP, kp += RPP, slot += RPP) {
            while (slot >= p.page_size) { slot -= p.page_size; ++blk; }
            bool valid = kp < kv_len;
            if (valid && blk != cur_blk) { page = bt[blk]; cur_blk = blk; }
            valid = valid && page >= 0 && page < p.num_pages;
            const size_t off = valid ? ((((size_t)page * p.nkv + g) * p.page_size + slot) * HD + ch * 8) : 0;
            cp_async16(smem_u32(k_tile + row * ROW_BYTES + ch * 16), p.k_pages + off, valid);
            cp_async16(smem_u32(v_tile + row * ROW_BYTES + ch * 16), p.v_pages + off, valid);
        }
    } else {
        for (int idx = threadIdx.x; idx < BN * CPR; idx += THREADS) {
            const int row = idx / CPR, ch = idx - row * CPR;
            const int kp = key0 + row;
            bool valid = kp < kv_len;
            int page = valid ? bt[kp / p.page_size] : -1;
            valid = valid && page >= 0 && page < p.num_pages;
            const size_t off = valid ? ((((size_t)page * p.nkv + g) * p.page_size + (kp % p.page_size)) * HD + ch * 8) : 0;
            cp_async16(smem_u32(k_tile + row * ROW_BYTES + ch * 16), p.k_pages + off, valid);
            cp_async16(smem_u32(v_tile + row * ROW_BYTES + ch * 16), p.v_pages + off, valid);
        }
    }
}

// Rows [row0, row0 + 16) of the stacked queries of (request, kv head g) into 16 padded smem rows
// (zeros for rows beyond n_rows).  row = token * G + head-in-group.
__device__ __forceinline__ void load_q_rows(const Params& p, int tok_base, int g, int row0, int n_rows,
                                            uint8_t* q_tile, int rows_to_load) {
    for (int idx = threadIdx.x; idx < rows_to_load * CPR; idx += THREADS) {
        const int r = idx / CPR, ch = idx - r * CPR;
        const int row = row0 + r;
        const bool valid = row < n_rows;
        const int tok = row / p.G, hg = row - tok * p.G;
        const size_t off = valid ? (((size_t)(tok_base + tok) * p.nh + g * p.G + hg) * HD + ch * 8) : 0;
        cp_async16(smem_u32(q_tile + r * ROW_BYTES + ch * 16), p.q + off, valid);
    }
}

struct RowState {
    float m[2], l[2];      // rows lane/4 and lane/4 + 8 of the warp's 16
    int qpos[2], lo[2];    // the rows' own positions and first visible key (qpos < 0: no such row)
};

// One slab of NK keys (starting k_off rows into the tiles) for the warp's 16 query rows.
template <int NK>
__device__ __forceinline__ void process_keys(const uint32_t (&qf)[KSTEPS][4], const uint8_t* k_tile,
                                             const uint8_t* v_tile, int k_off, int key_pos0, bool need_mask,
                                             float scale_log2, RowState& st, float (&o)[HD / 8][4]) {
    const int lane = threadIdx.x & 31;
    float s[NK / 8][4];
#pragma unroll
    for (int j = 0; j < NK / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
    const uint32_t kb = smem_u32(k_tile) + (k_off + (lane & 7) + 8 * (lane >> 4)) * ROW_BYTES + 16 * ((lane >> 3) & 1);
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
        for (int nb = 0; nb < NK / 16; ++nb) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4(kb + nb * 16 * ROW_BYTES + ks * 32, b0, b1, b2, b3);
            mma_bf16(s[2 * nb], qf[ks], b0, b1);
            mma_bf16(s[2 * nb + 1], qf[ks], b2, b3);
        }
    }
    // scale, mask, online softmax
    float mx[2] = {-INFINITY, -INFINITY};
    if (need_mask) {   // one branch per tile, not one per score
#pragma unroll
        for (int j = 0; j < NK / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = e >> 1;
                const int kp = key_pos0 + k_off + j * 8 + 2 * (lane & 3) + (e & 1);
                const float v = (kp > st.qpos[h] || kp < st.lo[h]) ? -INFINITY : s[j][e] * scale_log2;
                s[j][e] = v;
                mx[h] = fmaxf(mx[h], v);
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < NK / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float v = s[j][e] * scale_log2;
                s[j][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        }
    }
    float corr[2], mu[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(st.m[h], mx[h]);
        mu[h] = m_new == -INFINITY ? 0.f : m_new;
        corr[h] = exp2f(st.m[h] - mu[h]);   // m = -inf: 0
        st.m[h] = m_new;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < NK / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float pv = exp2f(s[j][e] - mu[e >> 1]);
            s[j][e] = pv;
            sum[e >> 1] += pv;
        }
    }
    st.l[0] = st.l[0] * corr[0] + sum[0];
    st.l[1] = st.l[1] * corr[1] + sum[1];
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) { o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1]; }
    // O += P . V
    const uint32_t vb = smem_u32(v_tile) + (k_off + (lane & 7) + 8 * ((lane >> 3) & 1)) * ROW_BYTES + 16 * (lane >> 4);
#pragma unroll
    for (int kk = 0; kk < NK / 16; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int nb = 0; nb < HD / 16; ++nb) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4_t(vb + kk * 16 * ROW_BYTES + nb * 32, b0, b1, b2, b3);
            mma_bf16(o[2 * nb], a, b0, b1);
            mma_bf16(o[2 * nb + 1], a, b2, b3);
        }
    }
}

__device__ __forceinline__ void load_q_frags(const uint8_t* q_rows, uint32_t (&qf)[KSTEPS][4]) {
    const int lane = threadIdx.x & 31;
    const uint32_t base = smem_u32(q_rows) + ((lane & 7) + 8 * ((lane >> 3) & 1)) * ROW_BYTES + 16 * (lane >> 4);
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) ldsm_x4(base + ks * 32, qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
}

__device__ __forceinline__ void init_rows(const Params& p, RowState& st, int row_base, int n_rows, int q_pos0) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = row_base + (lane >> 2) + 8 * h;
        st.m[h] = -INFINITY; st.l[h] = 0.f;
        if (row < n_rows) {
            st.qpos[h] = q_pos0 + row / p.G;
            st.lo[h] = p.window > 0 ? max(0, st.qpos[h] - p.window + 1) : 0;
        } else { st.qpos[h] = -1; st.lo[h] = 0; }
    }
}

// ---------------------------------------------------------------------------------------------
// work item: (request, first token of the tile within the request's segment, -, -)
__global__ void __launch_bounds__(THREADS)
attn_rows_kernel(Params p, int toks_per_tile) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    extern __shared__ __align__(16) uint8_t smem[];
    uint8_t* q_tile = smem;                       // 64 rows
    uint8_t* kv = smem + BN * ROW_BYTES;          // [2 stages][K, V]
    const int4 w = reinterpret_cast<const int4*>(p.work)[blockIdx.x];
    const int r = w.x, tok0 = w.y, g = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_len = p.cu_q[r + 1] - p.cu_q[r];
    const int kv_len = p.kv_len[r];
    const int ntok = min(toks_per_tile, q_len - tok0);
    const int n_rows = ntok * p.G;                // <= 64
    const int q_pos0 = p.q_start[r] + tok0;
    const int* bt = p.block_table + (size_t)r * p.max_blocks;

    load_q_rows(p, p.cu_q[r] + tok0, g, 0, n_rows, q_tile, 64);
    cp_async_commit();

    const int last_pos = q_pos0 + ntok - 1;
    const int first_key = p.window > 0 ? max(0, q_pos0 - p.window + 1) : 0;
    const int t_lo = first_key / BN, t_hi = last_pos / BN;   // inclusive
    load_kv_tile(p, bt, g, kv_len, t_lo * BN, kv, kv + TILE_BYTES);
    cp_async_commit();

    RowState st;
    init_rows(p, st, warp * 16, n_rows, q_pos0);
    float o[HD / 8][4];
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }

    cp_async_wait<1>();
    __syncthreads();
    uint32_t qf[KSTEPS][4];
    load_q_frags(q_tile + warp * 16 * ROW_BYTES, qf);
    const bool warp_live = warp * 16 < n_rows;
    const int warp_last_pos = q_pos0 + min(n_rows - 1, warp * 16 + 15) / p.G;

    for (int t = t_lo; t <= t_hi; ++t) {
        const int stage = (t - t_lo) & 1;
        uint8_t* k_tile = kv + stage * 2 * TILE_BYTES;
        if (t < t_hi) load_kv_tile(p, bt, g, kv_len, (t + 1) * BN, kv + (stage ^ 1) * 2 * TILE_BYTES,
                                   kv + (stage ^ 1) * 2 * TILE_BYTES + TILE_BYTES);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (warp_live && t * BN <= warp_last_pos) {
            const int warp_first_pos = q_pos0 + (warp * 16) / p.G;
            const bool need_mask = (t * BN + BN - 1 > warp_first_pos) ||
                                   (p.window > 0 && t * BN < warp_last_pos - p.window + 1);
            process_keys<BN>(qf, k_tile, k_tile + TILE_BYTES, 0, t * BN, need_mask, p.scale_log2, st, o);
        }
        __syncthreads();
    }
    // normalise and store
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float l = st.l[h];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const int row = warp * 16 + (lane >> 2) + 8 * h;
        if (row >= n_rows) continue;
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const int tok = row / p.G, hg = row - tok * p.G;
        bf16* dst = p.out + ((size_t)(p.cu_q[r] + tok0 + tok) * p.nh + g * p.G + hg) * HD + 2 * (lane & 3);
#pragma unroll
        for (int j = 0; j < HD / 8; ++j)
            *reinterpret_cast<__nv_bfloat162*>(dst + j * 8) =
                __floats2bfloat162_rn(o[j][2 * h] * inv, o[j][2 * h + 1] * inv);
    }
}

// Merges the four warps of a key-slice CTA (each saw a quarter of every tile's keys) through shared
// memory and writes the result: the final rows if the request has one slice, else this slice's
// partial sums.  `smem` may overlay the tiles: the caller's loop has ended.
__device__ __forceinline__ void finish_keys(const Params& p, const RowState& st, const float (&o)[HD / 8][4],
                                            uint8_t* smem, int r, int g, int slice, int n_slices, int item, int n_rows) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* ms = reinterpret_cast<float*>(smem);            // [4][16]
    float* ls = ms + NWARPS * 16;                          // [4][16]
    float* os = ls + NWARPS * 16;                          // [4][16][HD]
    sync_compute_warps();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float l = st.l[h];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const int row = (lane >> 2) + 8 * h;
        if ((lane & 3) == 0) { ms[warp * 16 + row] = st.m[h]; ls[warp * 16 + row] = l; }
#pragma unroll
        for (int j = 0; j < HD / 8; ++j) {
            float* d = os + ((size_t)(warp * 16 + row)) * HD + j * 8 + 2 * (lane & 3);
            d[0] = o[j][2 * h]; d[1] = o[j][2 * h + 1];
        }
    }
    sync_compute_warps();
    for (int idx = threadIdx.x; idx < n_rows * HD; idx += THREADS) {
        const int row = idx / HD, c = idx - row * HD;
        float M = -INFINITY;
#pragma unroll
        for (int wv = 0; wv < NWARPS; ++wv) M = fmaxf(M, ms[wv * 16 + row]);
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int wv = 0; wv < NWARPS; ++wv) {
            const float mw = ms[wv * 16 + row];
            const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
            acc += os[((size_t)(wv * 16 + row)) * HD + c] * f;
            L += ls[wv * 16 + row] * f;
        }
        const int tok = row / p.G, hg = row - tok * p.G;
        if (n_slices == 1) {
            p.out[((size_t)(p.cu_q[r] + tok) * p.nh + g * p.G + hg) * HD + c] =
                __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        } else {
            // `item` counts the slices of all earlier items, so every (item, kv head, slice) has its own slot
            const size_t pr = ((size_t)item * p.nkv + (size_t)g * n_slices + slice) * 16 + row;
            p.part_o[pr * HD + c] = acc;
            if (c == 0) { p.part_ml[pr * 2] = M; p.part_ml[pr * 2 + 1] = L; }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// work item: (request, slice, number of slices, item index for the partial buffers)
__global__ void __launch_bounds__(THREADS)
attn_keys_kernel(Params p) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    extern __shared__ __align__(16) uint8_t smem[];
    uint8_t* q_tile = smem;                       // 16 rows
    uint8_t* kv = smem + 16 * ROW_BYTES;          // [2 stages][K, V]
    const int4 w = reinterpret_cast<const int4*>(p.work)[blockIdx.x];
    const int r = w.x, slice = w.y, n_slices = w.z, item = w.w, g = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_len = p.cu_q[r + 1] - p.cu_q[r];
    const int kv_len = p.kv_len[r];
    const int n_rows = q_len * p.G;               // <= 16
    const int q_pos0 = p.q_start[r];
    const int* bt = p.block_table + (size_t)r * p.max_blocks;

    const int last_pos = q_pos0 + q_len - 1;
    const int first_key = p.window > 0 ? max(0, q_pos0 - p.window + 1) : 0;
    const int t_first = first_key / BN, t_end = last_pos / BN + 1;
    const int per = (t_end - t_first + n_slices - 1) / n_slices;
    const int t_lo = t_first + slice * per, t_hi = min(t_end, t_lo + per) - 1;   // inclusive; may be empty

    RowState st;
    init_rows(p, st, 0, n_rows, q_pos0);
    float o[HD / 8][4];
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }

    if (t_lo <= t_hi) {
        load_q_rows(p, p.cu_q[r], g, 0, n_rows, q_tile, 16);
        cp_async_commit();
        load_kv_tile(p, bt, g, kv_len, t_lo * BN, kv, kv + TILE_BYTES);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        uint32_t qf[KSTEPS][4];
        load_q_frags(q_tile, qf);
        for (int t = t_lo; t <= t_hi; ++t) {
            const int stage = (t - t_lo) & 1;
            uint8_t* k_tile = kv + stage * 2 * TILE_BYTES;
            if (t < t_hi) load_kv_tile(p, bt, g, kv_len, (t + 1) * BN, kv + (stage ^ 1) * 2 * TILE_BYTES,
                                       kv + (stage ^ 1) * 2 * TILE_BYTES + TILE_BYTES);
            cp_async_commit();
            cp_async_wait<1>();
            __syncthreads();
            const int k_off = warp * 16;
            if (t * BN + k_off <= last_pos) {
                const bool need_mask = (t * BN + BN - 1 > q_pos0) || (p.window > 0 && t * BN < last_pos - p.window + 1);
                process_keys<16>(qf, k_tile, k_tile + TILE_BYTES, k_off, t * BN, need_mask, p.scale_log2, st, o);
            }
            __syncthreads();
        }
    }
    finish_keys(p, st, o, smem, r, g, slice, n_slices, item, n_rows);
}

#if HEAD_DIM % 64 == 0
// ---------------------------------------------------------------------------------------------
// The same key-slice kernel with the K and V tiles brought in by TMA: one box per page and
// 128-byte column slice (a single instruction per 2 KB instead of 128 cp.async), 128-byte
// swizzle instead of padded rows, completion on an mbarrier.  Head sizes that are multiples of
// 64 and pages of 8, 16, 32 or 64 tokens.
constexpr int NSL = HD / 64;             // column slices
constexpr int SLICE_BYTES = BN * 128;    // one slice of a tile: 64 keys x 128 bytes
constexpr int TMA_TILE = NSL * SLICE_BYTES;

__device__ int g_tma_status = 0;

template <int NK>
__device__ __forceinline__ void process_keys_swz(const uint32_t (&qf)[KSTEPS][4], const uint8_t* k_tile,
                                                 const uint8_t* v_tile, int k_off, int key_pos0, bool need_mask,
                                                 float scale_log2, RowState& st, float (&o)[HD / 8][4]) {
    const int lane = threadIdx.x & 31, x7 = lane & 7;
    float s[NK / 8][4];
#pragma unroll
    for (int j = 0; j < NK / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
    // row & 7 == lane & 7 for every row this lane addresses (all other terms are multiples of 8)
    const uint32_t kb = smem_u32(k_tile) + (k_off + x7 + 8 * (lane >> 4)) * 128;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
        const int chunk = ks * 2 + ((lane >> 3) & 1);
        const uint32_t col = (chunk >> 3) * SLICE_BYTES + (((chunk & 7) ^ x7) << 4);
#pragma unroll
        for (int nb = 0; nb < NK / 16; ++nb) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4(kb + nb * 16 * 128 + col, b0, b1, b2, b3);
            mma_bf16(s[2 * nb], qf[ks], b0, b1);
            mma_bf16(s[2 * nb + 1], qf[ks], b2, b3);
        }
    }
    float mx[2] = {-INFINITY, -INFINITY};
    if (need_mask) {   // one branch per tile, not one per score
#pragma unroll
        for (int j = 0; j < NK / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = e >> 1;
                const int kp = key_pos0 + k_off + j * 8 + 2 * (lane & 3) + (e & 1);
                const float v = (kp > st.qpos[h] || kp < st.lo[h]) ? -INFINITY : s[j][e] * scale_log2;
                s[j][e] = v;
                mx[h] = fmaxf(mx[h], v);
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < NK / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float v = s[j][e] * scale_log2;
                s[j][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        }
    }
    float corr[2], mu[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(st.m[h], mx[h]);
        mu[h] = m_new == -INFINITY ? 0.f : m_new;
        corr[h] = exp2f(st.m[h] - mu[h]);
        st.m[h] = m_new;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < NK / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float pv = exp2f(s[j][e] - mu[e >> 1]);
            s[j][e] = pv;
            sum[e >> 1] += pv;
        }
    }
    st.l[0] = st.l[0] * corr[0] + sum[0];
    st.l[1] = st.l[1] * corr[1] + sum[1];
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) { o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1]; }
    const uint32_t vb = smem_u32(v_tile) + (k_off + x7 + 8 * ((lane >> 3) & 1)) * 128;
#pragma unroll
    for (int kk = 0; kk < NK / 16; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int nb = 0; nb < HD / 16; ++nb) {
            const int chunk = nb * 2 + (lane >> 4);
            const uint32_t col = (chunk >> 3) * SLICE_BYTES + (((chunk & 7) ^ x7) << 4);
            uint32_t b0, b1, b2, b3;
            ldsm_x4_t(vb + kk * 16 * 128 + col, b0, b1, b2, b3);
            mma_bf16(o[2 * nb], a, b0, b1);
            mma_bf16(o[2 * nb + 1], a, b2, b3);
        }
    }
}

constexpr int KEYS_TMA_TILES = 4 * TMA_TILE;                      // 2 stages of K and V
constexpr int KEYS_TMA_LOOP = KEYS_TMA_TILES + 16 * ROW_BYTES + 64 + 4 * HD + 1024;   // + query rows + barriers + the token's own key and value + alignment slack
constexpr int SMEM_KEYS_TMA = KEYS_TMA_LOOP > SMEM_KEYS_MERGE_BYTES + 1024 ? KEYS_TMA_LOOP : SMEM_KEYS_MERGE_BYTES + 1024;

// The decode token's query rows (the G heads of kv head g) from the unsummed q/k/v product, rotated, into
// the 16 padded rows of q_tile (the other rows zero); with want_kv also the token's rotated key and its value
// into kv_new [2][HD] (shared memory) and, if the token's page exists, into the cache.  A unit of work
// is two neighbouring floats of a head: a (channel j, channel j + rd / 2) pair of a q or k head, two
// channels in place elsewhere; four units a thread and four planes at a time are in flight together.
__device__ __forceinline__ void rows_from_qkv(const Params& p, int tok, int g, int pos, const int* bt,
                                              uint8_t* q_tile, bf16* kv_new, bool want_kv) {
    const int half = p.rd >> 1;
    const size_t width = (size_t)(p.nh + 2 * p.nkv) * HD;
    const float* row = p.qkv + (size_t)tok * width;
    const float* tab = p.rope_table + (size_t)tok * p.rd;
    const int units = (p.G + (want_kv ? 2 : 0)) * (HD / 2);
    bf16* k_dst = nullptr; bf16* v_dst = nullptr;
    if (want_kv) {
        const int page = bt[pos / p.page_size];
        if (page >= 0 && page < p.num_pages) {
            const size_t at = (((size_t)page * p.nkv + g) * p.page_size + pos % p.page_size) * HD;
            k_dst = const_cast<bf16*>(p.k_pages) + at; v_dst = const_cast<bf16*>(p.v_pages) + at;
        }
    }
    for (int idx = threadIdx.x; idx < (16 - p.G) * CPR; idx += THREADS)   // rows that hold no query
        *reinterpret_cast<uint4*>(q_tile + (p.G + idx / CPR) * ROW_BYTES + (idx % CPR) * 16) = make_uint4(0, 0, 0, 0);
    for (int u0 = threadIdx.x; u0 < units; u0 += 4 * THREADS) {
        const float* src[4];
        float2 acc[4];
        float cs[4], sn[4];
        int hs[4], j[4];
        bool rot[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int u = u0 + i * THREADS;
            hs[i] = u < units ? u / (HD / 2) : -1;
            j[i] = u - (u / (HD / 2)) * (HD / 2);
            const int head = hs[i] < p.G ? g * p.G + hs[i] : (hs[i] == p.G ? p.nh + g : p.nh + p.nkv + g);
            src[i] = row + (size_t)head * HD + 2 * j[i];
            rot[i] = hs[i] >= 0 && hs[i] <= p.G && 2 * j[i] < p.rd;      // a q or k head's rotated pair
            acc[i] = make_float2(0.f, 0.f);
            cs[i] = rot[i] ? tab[j[i]] : 1.f;
            sn[i] = rot[i] ? tab[half + j[i]] : 0.f;
        }
        for (int p0 = 0; p0 < p.qkv_planes; p0 += 4) {
            float2 t[4][4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    t[q][i] = (hs[i] >= 0 && p0 + q < p.qkv_planes)
                        ? *reinterpret_cast<const float2*>(src[i] + (size_t)(p0 + q) * p.qkv_plane_stride) : make_float2(0.f, 0.f);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
#pragma unroll
                for (int i = 0; i < 4; ++i) { acc[i].x += t[q][i].x; acc[i].y += t[q][i].y; }
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (hs[i] < 0) continue;
            // x cos - partner sin for the first half's channel, x cos + partner sin for the second's
            const float a = rot[i] ? acc[i].x * cs[i] + acc[i].y * -sn[i] : acc[i].x;
            const float b = rot[i] ? acc[i].y * cs[i] + acc[i].x * sn[i] : acc[i].y;
            const int c0 = rot[i] ? j[i] : 2 * j[i], c1 = rot[i] ? j[i] + half : 2 * j[i] + 1;
            const bf16 va = __float2bfloat16_rn(a), vb = __float2bfloat16_rn(b);
            if (hs[i] < p.G) {
                bf16* qr = reinterpret_cast<bf16*>(q_tile + hs[i] * ROW_BYTES);
                qr[c0] = va; qr[c1] = vb;
            } else {
                bf16* st = kv_new + (hs[i] - p.G) * HD;
                st[c0] = va; st[c1] = vb;
                bf16* dst = hs[i] == p.G ? k_dst : v_dst;
                if (dst) { dst[c0] = va; dst[c1] = vb; }
            }
        }
    }
}

// Warp 0 issues the boxes of the next tile while all four warps work on the current one.  (A
// separate producer warp with deeper stages was measured slower: its registers cost the third
// CTA per SM, and this kernel lives on the number of warps in flight.)
__global__ void __launch_bounds__(THREADS)
attn_keys_tma_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, Params p) {
    BW_PDL_TRIGGER();
    extern __shared__ __align__(16) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* kv = smem;                           // [2 stages][K tile, V tile], each 1024-aligned (swizzle)
    uint8_t* q_tile = smem + KEYS_TMA_TILES;      // 16 padded rows
    uint64_t* bars = reinterpret_cast<uint64_t*>(q_tile + 16 * ROW_BYTES);
    bf16* kv_new = reinterpret_cast<bf16*>(q_tile + 16 * ROW_BYTES + 64);   // [2][HD]: the token's own key and value
    const uint32_t full0 = smem_u32(bars);
    if (threadIdx.x == 0) {
        bw::mbar_init(full0, 1); bw::mbar_init(full0 + 8, 1);
        bw::fence_barrier_init();
        bw::tma_prefetch_desc(&tmK); bw::tma_prefetch_desc(&tmV);
    }
    __syncthreads();
    // The step's lists (work items, lengths, block tables) were on the device before the step's first
    // kernel ran; only the queries, and the keys and values of this step's own tokens, come from the
    // kernels just before this one.  The wait for those kernels therefore comes late (below).
    const int4 w = reinterpret_cast<const int4*>(p.work)[blockIdx.x];
    const int r = w.x, slice = w.y, n_slices = w.z, item = w.w, g = blockIdx.y;
    const int warp = threadIdx.x >> 5;
    const int q_len = p.cu_q[r + 1] - p.cu_q[r];
    const int kv_len = p.kv_len[r];
    const int n_rows = q_len * p.G;               // <= 16
    const int q_pos0 = p.q_start[r];
    const int* bt = p.block_table + (size_t)r * p.max_blocks;
    const int last_pos = q_pos0 + q_len - 1;
    const int first_key = p.window > 0 ? max(0, q_pos0 - p.window + 1) : 0;
    const int t_first = first_key / BN, t_end = last_pos / BN + 1;
    const int per = (t_end - t_first + n_slices - 1) / n_slices;
    const int t_lo = t_first + slice * per, t_hi = min(t_end, t_lo + per) - 1;   // inclusive; may be empty
    const int ppt = BN / p.page_size;

    // Warp 0 feeds the tiles: lane pg owns page pg of a tile.  Its page id is looked up one tile
    // before its boxes are issued, so the lookup's latency is off the path; pages that do not
    // exist are skipped (the warps clear their rows).
    const int lane = threadIdx.x & 31;
    int my_page = -1;
    auto lookup = [&](int t) {
        const int key = t * BN + lane * p.page_size;
        const int page = (lane < ppt && t <= t_hi && key < kv_len) ? bt[key / p.page_size] : -1;
        my_page = page < p.num_pages ? page : -1;
    };
    auto issue_tile = [&](int stage) {
        uint8_t* k_tile = kv + stage * 2 * TMA_TILE;
        const int n_ok = __popc(__ballot_sync(0xffffffffu, my_page >= 0));
        const uint32_t bar = full0 + 8 * stage;
        if (lane == 0) bw::mbar_expect_tx(bar, n_ok * 2 * NSL * p.page_size * 128);
        __syncwarp();
        if (my_page >= 0) {
            const int y = (my_page * p.nkv + g) * p.page_size;
            const uint32_t off = lane * p.page_size * 128;
#pragma unroll
            for (int h = 0; h < NSL; ++h) {
                bw::tma_load_2d(smem_u32(k_tile + h * SLICE_BYTES + off), &tmK, bar, h * 64, y);
                bw::tma_load_2d(smem_u32(k_tile + TMA_TILE + h * SLICE_BYTES + off), &tmV, bar, h * 64, y);
            }
        }
    };

    RowState st;
    init_rows(p, st, 0, n_rows, q_pos0);
    float o[HD / 8][4];
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }

    // a first tile that holds none of this step's tokens is requested before the wait
    const bool early = t_lo <= t_hi && t_lo * BN + BN <= q_pos0;
    if (early && warp == 0) { lookup(t_lo); issue_tile(0); lookup(t_lo + 1); }
    BW_PDL_WAIT();
    // from the unsummed q/k/v product: the slice that holds the token's own position (one per request and
    // kv head, never empty) also makes the token's key and value and puts them into its tile below
    const int t_own = last_pos / BN;
    const bool own = p.qkv != nullptr && p.append && t_lo <= t_own && t_own <= t_hi;
    if (t_lo <= t_hi) {
        if (!early && warp == 0) { lookup(t_lo); issue_tile(0); lookup(t_lo + 1); }
        if (p.qkv) {
            rows_from_qkv(p, p.cu_q[r], g, last_pos, bt, q_tile, kv_new, own);
        } else {
            load_q_rows(p, p.cu_q[r], g, 0, n_rows, q_tile, 16);
            cp_async_commit();
            cp_async_wait<0>();
        }
        __syncthreads();
        uint32_t qf[KSTEPS][4];
        load_q_frags(q_tile, qf);
        bool ok = true;
        for (int t = t_lo; t <= t_hi && ok; ++t) {
            const int i = t - t_lo, stage = i & 1;
            uint8_t* k_tile = kv + stage * 2 * TMA_TILE;
            uint8_t* v_tile = k_tile + TMA_TILE;
            if (warp == 0 && t < t_hi) { issue_tile(stage ^ 1); lookup(t + 2); }
            ok = bw::mbar_wait(full0 + 8 * stage, (i >> 1) & 1, &g_tma_status, 21);
            if (own && t == t_own) {
                // the cache's row of the token's own position was loaded as it was before this step: the
                // key and value made above take its place (swizzled like the boxes around it)
                const int rk = last_pos - t * BN;
                for (int idx = threadIdx.x; idx < 2 * CPR; idx += THREADS) {
                    const int which = idx / CPR, ch = idx - which * CPR;
                    uint8_t* tile = which ? v_tile : k_tile;
                    *reinterpret_cast<uint4*>(tile + (ch >> 3) * SLICE_BYTES + rk * 128 + (((ch & 7) ^ (rk & 7)) << 4)) =
                        *reinterpret_cast<const uint4*>(kv_new + which * HD + ch * 8);
                }
                __syncthreads();
            }
            // Rows of keys that do not exist hold whatever was there: values times a probability of
            // 0 must still be 0, so those rows of V are cleared (only in a request's last tile or at
            // a window's edge).
            if (t * BN + BN > kv_len || (p.window > 0 && t * BN < first_key)) {
                for (int idx = threadIdx.x; idx < BN * NSL * 8; idx += THREADS) {
                    const int rk = idx / (NSL * 8), rem = idx - rk * (NSL * 8);
                    const int key = t * BN + rk;
                    if (key >= kv_len || bt[key / p.page_size] < 0)
                        *reinterpret_cast<uint4*>(v_tile + (rem >> 3) * SLICE_BYTES + rk * 128 + (rem & 7) * 16) = make_uint4(0, 0, 0, 0);
                }
                __syncthreads();
            }
            const int k_off = warp * 16;
            if (ok && t * BN + k_off <= last_pos) {
                const bool need_mask = (t * BN + BN - 1 > q_pos0) || (p.window > 0 && t * BN < last_pos - p.window + 1);
                process_keys_swz<16>(qf, k_tile, v_tile, k_off, t * BN, need_mask, p.scale_log2, st, o);
            }
            // every warp is done with this stage before it is loaded again; a timeout ends the loop for all
            ok = __syncthreads_and(ok) != 0;
        }
    }
    __syncthreads();
    finish_keys(p, st, o, smem, r, g, slice, n_slices, item, n_rows);
}
#endif  // HEAD_DIM % 64 == 0

// Sums the slices of every sliced item: grid (sliced items, nkv, 16 rows), one row of one head per
// CTA.  The threads form MERGE_GROUPS groups of HD / 4; group j takes slices j, j + MERGE_GROUPS, ...
// with one float4 each, so all loads of a row are in flight together; shared memory adds the groups
// (in slice order within a group, groups in order: the same sum whatever ran beside it).
constexpr int MAX_SLICES = 64;
constexpr int MERGE_THREADS = 256;
constexpr int MERGE_QUADS = HD / 4;
constexpr int MERGE_GROUPS = MERGE_THREADS / MERGE_QUADS < MAX_SLICES ? MERGE_THREADS / MERGE_QUADS : MAX_SLICES;
constexpr int MERGE_PER = (MAX_SLICES + MERGE_GROUPS - 1) / MERGE_GROUPS;
__global__ void __launch_bounds__(MERGE_THREADS)
attn_merge_kernel(Params p, const int* merge_items) {
    BW_PDL_TRIGGER();
    const int4 w = reinterpret_cast<const int4*>(merge_items)[blockIdx.x];   // written before the step's first kernel
    const int r = w.x, n_slices = w.z, item = w.w, g = blockIdx.y, row = blockIdx.z;
    BW_PDL_WAIT();
    const int n_rows = (p.cu_q[r + 1] - p.cu_q[r]) * p.G;
    if (row >= n_rows) return;
    __shared__ float sm_m[MAX_SLICES], sm_f[MAX_SLICES], sm_lf[MAX_SLICES];
    __shared__ float4 red[MERGE_GROUPS][MERGE_QUADS];
    const size_t base0 = ((size_t)item * p.nkv + (size_t)g * n_slices) * 16 + row;
    const int tid = threadIdx.x, quad = tid % MERGE_QUADS, group = tid / MERGE_QUADS;
    // this thread's partial outputs: issued before anything that depends on the maxima
    float4 part[MERGE_PER];
    if (group < MERGE_GROUPS) {
#pragma unroll
        for (int i = 0; i < MERGE_PER; ++i) {
            const int sl = group + i * MERGE_GROUPS;
            part[i] = sl < n_slices ? reinterpret_cast<const float4*>(p.part_o + (base0 + (size_t)sl * 16) * HD)[quad]
                                    : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    float l_mine = 0.f;
    if (tid < n_slices) {
        const float2 ml = reinterpret_cast<const float2*>(p.part_ml)[base0 + (size_t)tid * 16];
        sm_m[tid] = ml.x; l_mine = ml.y;
    }
    __syncthreads();
    float M = -INFINITY;
    for (int sl = 0; sl < n_slices; ++sl) M = fmaxf(M, sm_m[sl]);
    if (tid < n_slices) {
        const float f = sm_m[tid] == -INFINITY ? 0.f : exp2f(sm_m[tid] - M);
        sm_f[tid] = f; sm_lf[tid] = l_mine * f;
    }
    __syncthreads();
    if (group < MERGE_GROUPS) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < MERGE_PER; ++i) {
            const int sl = group + i * MERGE_GROUPS;
            if (sl < n_slices) {
                const float f = sm_f[sl];
                acc.x += part[i].x * f; acc.y += part[i].y * f; acc.z += part[i].z * f; acc.w += part[i].w * f;
            }
        }
        red[group][quad] = acc;
    }
    __syncthreads();
    if (tid < MERGE_QUADS) {
        float4 acc = red[0][tid];
        for (int j = 1; j < MERGE_GROUPS; ++j) {
            const float4 v = red[j][tid];
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        float L = 0.f;
        for (int sl = 0; sl < n_slices; ++sl) L += sm_lf[sl];
        const float inv = L > 0.f ? 1.f / L : 0.f;
        const int tok = row / p.G, hg = row - tok * p.G;
        bf16* dst = p.out + ((size_t)(p.cu_q[r] + tok) * p.nh + g * p.G + hg) * HD + tid * 4;
        const uint2 packed = make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
        *reinterpret_cast<uint2*>(dst) = packed;
    }
}

// The same for items of at most MERGE_FEW slices (decode batches of several requests, where the slices are few): one CTA per
// (item, kv head), a thread per row and four channels; every thread fetches the maxima and sums of its
// row's slices itself, so all its loads are in flight together and nothing waits at a barrier.
#ifndef ATTN_MERGE_FEW
#define ATTN_MERGE_FEW 8   // measured: 1 % of a decode step at batch 8 (6 slices); 16 gains nothing at 6 and loses at 13 slices
#endif
constexpr int MERGE_FEW = ATTN_MERGE_FEW;
__global__ void __launch_bounds__(16 * MERGE_QUADS)
attn_merge_few_kernel(Params p, const int* merge_items) {
    BW_PDL_TRIGGER();
    const int4 w = reinterpret_cast<const int4*>(merge_items)[blockIdx.x];
    const int r = w.x, n_slices = w.z, item = w.w, g = blockIdx.y;
    const int row = threadIdx.x / MERGE_QUADS, quad = threadIdx.x - row * MERGE_QUADS;
    BW_PDL_WAIT();
    const int n_rows = (p.cu_q[r + 1] - p.cu_q[r]) * p.G;
    if (row >= n_rows) return;
    const size_t base0 = ((size_t)item * p.nkv + (size_t)g * n_slices) * 16 + row;
    float4 part[MERGE_FEW];
    float2 ml[MERGE_FEW];
#pragma unroll
    for (int sl = 0; sl < MERGE_FEW; ++sl) {
        const bool there = sl < n_slices;
        ml[sl] = there ? reinterpret_cast<const float2*>(p.part_ml)[base0 + (size_t)sl * 16] : make_float2(-INFINITY, 0.f);
        part[sl] = there ? reinterpret_cast<const float4*>(p.part_o + (base0 + (size_t)sl * 16) * HD)[quad]
                         : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float M = -INFINITY;
#pragma unroll
    for (int sl = 0; sl < MERGE_FEW; ++sl) M = fmaxf(M, ml[sl].x);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float L = 0.f;
#pragma unroll
    for (int sl = 0; sl < MERGE_FEW; ++sl) {
        const float f = ml[sl].x == -INFINITY ? 0.f : exp2f(ml[sl].x - M);
        acc.x += part[sl].x * f; acc.y += part[sl].y * f; acc.z += part[sl].z * f; acc.w += part[sl].w * f;
        L += ml[sl].y * f;
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    const int tok = row / p.G, hg = row - tok * p.G;
    bf16* dst = p.out + ((size_t)(p.cu_q[r] + tok) * p.nh + g * p.G + hg) * HD + quad * 4;
    *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
}

constexpr int SMEM_ROWS = (BN + 4 * BN) * ROW_BYTES;     // q tile of 64 rows + 2 stages of K and V
constexpr int SMEM_KEYS_LOOP = (16 + 4 * BN) * ROW_BYTES;
constexpr int SMEM_KEYS_MERGE = SMEM_KEYS_MERGE_BYTES;
constexpr int SMEM_KEYS = SMEM_KEYS_LOOP > SMEM_KEYS_MERGE ? SMEM_KEYS_LOOP : SMEM_KEYS_MERGE;

}  // namespace

BW_EXPORT int bw_attention_head_dim() { return HD; }

// rows_work: n_rows_items int4 (request, first token, 0, 0) for segments of more than 16 stacked rows.
// keys_work: n_keys_items int4 (request, slice, slices, item) for the others; merge_work: one int4 per
// item that has more than one slice (merge_max_slices: the most slices any of them has, 0: unknown).
// part_o / part_ml: float32 scratch for
// [items, nkv, slices, 16, HD] and [.., 2].  window <= 0: all keys.
// qkv != null (q may be null then): every request has ONE token, and its queries, key and value come from
// the q/k/v product itself: float32 [qkv_planes][tokens][(nh + 2 nkv) * HD], the planes qkv_plane_stride
// floats apart and added in order, the rotated channels of the q and k heads as (j, j + rd / 2) pairs;
// rope_table float32 [tokens][rd] (cosines, then sines); append != 0: key and value also go to the cache.
// Only where the TMA key-slice kernel runs (head size a multiple of 64, pages of 8 to 64 tokens);
// BW_ERR_UNSUPPORTED otherwise, and nothing was launched.
BW_EXPORT int bw_attention_mma(const void* q, const void* k_pages, const void* v_pages, void* out, const int* cu_q,
                               const int* q_start, const int* kv_len, const int* block_table, int max_blocks,
                               const int* rows_work, int n_rows_items, const int* keys_work, int n_keys_items,
                               const int* merge_work, int n_merge_items, float* part_o, float* part_ml, int nh,
                               int nkv, int page_size, int num_pages, int window, float scale,
                               const float* qkv, int qkv_planes, long long qkv_plane_stride, const float* rope_table,
                               int rd, int append, int merge_max_slices, void* stream) {
    if (nkv <= 0 || nh % nkv != 0) return BW_ERR_BAD_ARG;
    const int G = nh / nkv;
    if (G > 16) return BW_ERR_UNSUPPORTED;
    const bool tma_keys = HD % 64 == 0 && (page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64) &&
                          (((uintptr_t)k_pages | (uintptr_t)v_pages) & 15) == 0;
    if (qkv) {
        if (!tma_keys) return BW_ERR_UNSUPPORTED;
        if (n_rows_items > 0 || qkv_planes < 1 || rd < 0 || rd > HD || (rd & 1) || (rd > 0 && !rope_table) ||
            (((uintptr_t)qkv | (uintptr_t)(qkv_plane_stride * 4)) & 7))
            return BW_ERR_BAD_ARG;
    } else if (!q) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    static bool rows_attr_done[bw::MAX_DEVICES], keys_attr_done[bw::MAX_DEVICES];
    if (cudaError_t e = bw::allow_dynamic_smem(attn_rows_kernel, SMEM_ROWS, rows_attr_done); e != cudaSuccess) return (int)e;
    if (cudaError_t e = bw::allow_dynamic_smem(attn_keys_kernel, SMEM_KEYS, keys_attr_done); e != cudaSuccess) return (int)e;
    Params p;
    p.q = (const bf16*)q; p.k_pages = (const bf16*)k_pages; p.v_pages = (const bf16*)v_pages; p.out = (bf16*)out;
    p.cu_q = cu_q; p.q_start = q_start; p.kv_len = kv_len; p.block_table = block_table;
    p.part_o = part_o; p.part_ml = part_ml;
    p.max_blocks = max_blocks; p.nh = nh; p.nkv = nkv; p.G = G; p.page_size = page_size; p.num_pages = num_pages;
    p.window = window > 0 ? window : 0;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.qkv = qkv; p.qkv_plane_stride = qkv_plane_stride; p.rope_table = rope_table;
    p.qkv_planes = qkv_planes; p.rd = rd; p.append = append;
    if (n_rows_items > 0) {
        p.work = rows_work;
        bw::launch((attn_rows_kernel), dim3(dim3(n_rows_items, nkv)), dim3(THREADS), SMEM_ROWS, s, p, 64 / G);
        BW_LAUNCH_CHECK();
    }
    if (n_keys_items > 0) {
        p.work = keys_work;
        bool launched = false;
#if HEAD_DIM % 64 == 0
        if (tma_keys) {
            static bool tma_attr_done[bw::MAX_DEVICES];
            if (cudaError_t e = bw::allow_dynamic_smem(attn_keys_tma_kernel, SMEM_KEYS_TMA, tma_attr_done); e != cudaSuccess) return (int)e;
            CUtensorMap tk, tv;
            cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)num_pages * nkv * page_size};
            cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
            cuuint32_t box[2] = {64, (cuuint32_t)page_size};
            if (!bw::encode_bf16_sw128(&tk, k_pages, 2, dims, strides, box) ||
                !bw::encode_bf16_sw128(&tv, v_pages, 2, dims, strides, box))
                return BW_ERR_DRIVER;
            bw::launch((attn_keys_tma_kernel), dim3(n_keys_items, nkv), dim3(THREADS), SMEM_KEYS_TMA, s, tk, tv, p);
            BW_LAUNCH_CHECK();
            launched = true;
        }
#endif
        if (!launched) {
            bw::launch((attn_keys_kernel), dim3(dim3(n_keys_items, nkv)), dim3(THREADS), SMEM_KEYS, s, p);
            BW_LAUNCH_CHECK();
        }
        if (n_merge_items > 0) {
            // merge_max_slices: the most slices of any merge item (0: unknown)
            if (merge_max_slices > 0 && merge_max_slices <= MERGE_FEW && 16 * MERGE_QUADS <= 1024)
                bw::launch((attn_merge_few_kernel), dim3(n_merge_items, nkv), dim3(16 * MERGE_QUADS), 0, s, p, merge_work);
            else
                bw::launch((attn_merge_kernel), dim3(n_merge_items, nkv, 16), dim3(MERGE_THREADS), 0, s, p, merge_work);
            BW_LAUNCH_CHECK();
        }
    }
    return 0;
}
