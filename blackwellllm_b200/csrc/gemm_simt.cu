// out[M,N] (=|+=) x[M,K] . w[N,K]^T (+ bias[N])  on the CUDA cores with float32
// fused multiply-adds: the true 32-bit matrix product (no tensor cores, no reduced
// precision mode).  It is also the fallback for bfloat16 shapes the tensor-core
// kernel refuses (K not a multiple of 8).  Any M, N, K.
//
// Each output element is the sum over k in ascending order of 16-wide slices, so a
// row's result does not depend on what other rows are in the batch.
#include "common.cuh"

using bf16 = __nv_bfloat16;

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename XT, typename WT, typename BT, typename OT, bool ACCUM>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const XT* __restrict__ x, const WT* __restrict__ w, const BT* __restrict__ bias,
                 OT* __restrict__ out, int M, int N, int K, int ldx, int ldo) {
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, each TM x TN outputs
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    // each thread loads 4 elements of each tile per slice: row = tid / 4, k = (tid % 4) * 4 ..+3
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int k = k0 + lk + q;
            const int gm = m0 + lr, gn = n0 + lr;
            xs[lk + q][lr] = (gm < M && k < K) ? bw::to_f32(x[(size_t)gm * ldx + k]) : 0.f;
            ws[lk + q][lr] = (gn < N && k < K) ? bw::to_f32(w[(size_t)gn * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = xs[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (bias) v += bw::to_f32(bias[gn]);
            OT* o = out + (size_t)gm * ldo + gn;
            if (ACCUM) v += bw::to_f32(*o);
            *o = bw::from_f32<OT>(v);
        }
    }
}

template <typename XT, typename WT, typename OT>
int launch(const void* x, const void* w, const void* bias, int bias_type, void* out, int M, int N, int K,
           int ldx, int ldo, int accumulate, cudaStream_t s) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    const XT* xp = (const XT*)x; const WT* wp = (const WT*)w; OT* op = (OT*)out;
#define BW_GO(BT, ACC) gemm_simt_kernel<XT, WT, BT, OT, ACC><<<grid, 256, 0, s>>>(xp, wp, (const BT*)bias, op, M, N, K, ldx, ldo)
    if (bias && bias_type == BW_BF16) { if (accumulate) BW_GO(bf16, true); else BW_GO(bf16, false); }
    else { if (accumulate) BW_GO(float, true); else BW_GO(float, false); }
#undef BW_GO
    BW_LAUNCH_CHECK();
    return 0;
}

}  // namespace

// in_type: type of x and w (both the same); out_type: type of out.
// accumulate != 0: out += product (out must be float32: the residual stream).
BW_EXPORT int bw_gemm_simt(const void* x, const void* w, int in_type, const void* bias, int bias_type,
                           void* out, int out_type, int M, int N, int K, int ldx, int ldo,
                           int accumulate, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || ldx < K || ldo < N) return BW_ERR_BAD_ARG;
    if (accumulate && out_type != BW_F32) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (in_type == BW_F32 && out_type == BW_F32)
        return launch<float, float, float>(x, w, bias, bias_type, out, M, N, K, ldx, ldo, accumulate, s);
    if (in_type == BW_BF16 && out_type == BW_F32)
        return launch<bf16, bf16, float>(x, w, bias, bias_type, out, M, N, K, ldx, ldo, accumulate, s);
    if (in_type == BW_BF16 && out_type == BW_BF16)
        return launch<bf16, bf16, bf16>(x, w, bias, bias_type, out, M, N, K, ldx, ldo, accumulate, s);
    return BW_ERR_BAD_ARG;
}
