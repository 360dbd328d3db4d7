// Paged causal grouped-query attention on the CUDA cores, all arithmetic float32.
// This is the attention of the true 32-bit path, and the plain twin that the
// tensor-core attention kernel is tested against.  One block (4 warps) per
// (token, query head); it takes any mix of prompt portions and decode tokens,
// because every token carries its own position and request.
//
// Keys are visited in 32-key chunks; chunk i belongs to warp i % 4, and the four
// partial results are merged in warp order.  The order of the sums is therefore a
// function of the key positions alone, never of the batch.
#include "common.cuh"

using bf16 = __nv_bfloat16;

namespace {

constexpr int WARPS = 4;
constexpr int MAX_CH = 8;  // channels per lane: head_dim <= 256

template <typename QT, typename KT, typename OT>
__global__ void __launch_bounds__(WARPS * 32)
attention_simt_kernel(const QT* __restrict__ q, const KT* __restrict__ k_pages,
                      const KT* __restrict__ v_pages, const int* __restrict__ positions,
                      const int* __restrict__ req_of_token, const int* __restrict__ block_table,
                      int max_blocks, OT* __restrict__ out, int nh, int nkv, int hd, int page_size,
                      int num_pages, int window, float scale) {
    extern __shared__ float smem[];
    float* qs = smem;                       // [hd]
    float* accs = qs + hd;                  // [WARPS][hd]
    float* ml = accs + WARPS * hd;          // [WARPS][2]
    const int t = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kvh = h / (nh / nkv);
    const int q_pos = positions[t];
    const int r = req_of_token[t];
    const int* bt = block_table + (size_t)r * max_blocks;
    const int lo = (window > 0 && q_pos - window + 1 > 0) ? q_pos - window + 1 : 0;
    const int n_keys = q_pos - lo + 1;

    for (int c = threadIdx.x; c < hd; c += blockDim.x)
        qs[c] = bw::to_f32(q[((size_t)t * nh + h) * hd + c]);
    __syncthreads();

    float m = -INFINITY, l = 0.f;
    float acc[MAX_CH];
#pragma unroll
    for (int i = 0; i < MAX_CH; ++i) acc[i] = 0.f;

    const int n_chunks = (n_keys + 31) / 32;
    for (int ch = warp; ch < n_chunks; ch += WARPS) {
        const int kp = lo + ch * 32 + lane;          // this lane's key position
        const bool valid = kp <= q_pos;
        float s = -INFINITY;
        size_t row_off = 0;
        if (valid) {
            const int page = bt[kp / page_size];
            if (page >= 0 && page < num_pages) {
                row_off = (((size_t)page * nkv + kvh) * page_size + (kp % page_size)) * hd;
                const KT* kr = k_pages + row_off;
                float d = 0.f;
                for (int c = 0; c < hd; ++c) d = fmaf(qs[c], bw::to_f32(kr[c]), d);
                s = d * scale;
            }
        }
        const float cm = bw::warp_max(s);
        const float m_new = fmaxf(m, cm);
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
        l = l * corr + bw::warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < MAX_CH; ++i) acc[i] *= corr;
        for (int j = 0; j < 32; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const size_t off = (size_t)__shfl_sync(0xffffffffu, (unsigned long long)row_off, j);
            if (pj == 0.f) continue;   // masked or beyond the last key (uniform across the warp)
            const KT* vr = v_pages + off;
#pragma unroll
            for (int i = 0; i < MAX_CH; ++i) {
                const int c = lane + 32 * i;
                if (c < hd) acc[i] = fmaf(pj, bw::to_f32(vr[c]), acc[i]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < MAX_CH; ++i) {
        const int c = lane + 32 * i;
        if (c < hd) accs[warp * hd + c] = acc[i];
    }
    if (lane == 0) { ml[warp * 2] = m; ml[warp * 2 + 1] = l; }
    __syncthreads();
    // merge the warps' partial softmaxes in warp order
    float M = -INFINITY;
    for (int w = 0; w < WARPS; ++w) M = fmaxf(M, ml[w * 2]);
    float L = 0.f;
    float f[WARPS];
    for (int w = 0; w < WARPS; ++w) {
        f[w] = (ml[w * 2] == -INFINITY) ? 0.f : expf(ml[w * 2] - M);
        L += ml[w * 2 + 1] * f[w];
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    for (int c = threadIdx.x; c < hd; c += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < WARPS; ++w) o += accs[w * hd + c] * f[w];
        out[((size_t)t * nh + h) * hd + c] = bw::from_f32<OT>(o * inv);
    }
}

}  // namespace

// type: element type of q, the pages and out (all the same).  window <= 0: all keys.
BW_EXPORT int bw_attention_simt(const void* q, const void* k_pages, const void* v_pages, int type,
                                const int* positions, const int* req_of_token, const int* block_table,
                                int max_blocks, void* out, int T, int nh, int nkv, int hd, int page_size,
                                int num_pages, int window, float scale, void* stream) {
    if (T <= 0) return 0;
    if (hd <= 0 || hd > 32 * MAX_CH || nkv <= 0 || nh % nkv != 0) return BW_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(T, nh);
    const size_t smem = (size_t)(hd + WARPS * hd + WARPS * 2) * sizeof(float);
    if (type == BW_F32)
        attention_simt_kernel<float, float, float><<<grid, WARPS * 32, smem, s>>>(
            (const float*)q, (const float*)k_pages, (const float*)v_pages, positions, req_of_token,
            block_table, max_blocks, (float*)out, nh, nkv, hd, page_size, num_pages, window, scale);
    else if (type == BW_BF16)
        attention_simt_kernel<bf16, bf16, bf16><<<grid, WARPS * 32, smem, s>>>(
            (const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, positions, req_of_token,
            block_table, max_blocks, (bf16*)out, nh, nkv, hd, page_size, num_pages, window, scale);
    else return BW_ERR_BAD_ARG;
    BW_LAUNCH_CHECK();
    return 0;
}
