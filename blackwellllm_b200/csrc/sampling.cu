// Token choice from float32 logits [R, V], one block per row.
//
//  * temperature <= 0: argmax, the lowest index winning a tie.
//  * temperature  > 0: softmax(logits / temperature) in float32; optional nucleus
//    (top_p < 1): keep the most probable tokens whose mass reaches top_p (all
//    tokens tied with the last one kept are kept too); then the inverse CDF over
//    the kept tokens IN INDEX ORDER at the uniform number u[r] given by the host.
//    The draw therefore depends on (logits row, u) only, not on the batch.
//
// Beside it: the repetition penalty on a row's logits before the choice, and the log
// probability of a given token (the reference's src/kernels/sampling.cu:85-118 and 213-247).
#include "common.cuh"

namespace {

constexpr int THREADS = 1024;

__device__ __forceinline__ void argmax_pair(float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

__device__ int block_argmax(const float* row, int V, float* sv, int* si) {
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int c = threadIdx.x; c < V; c += blockDim.x) {
        const float v = row[c];
        if (v > bv || (v == bv && c < bi)) { bv = v; bi = c; }
    }
    if (bi == 0x7fffffff) { bi = (int)threadIdx.x < V ? (int)threadIdx.x : 0; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        argmax_pair(bv, bi, ov, oi);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        bv = lane < nw ? sv[lane] : -INFINITY;
        bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            argmax_pair(bv, bi, ov, oi);
        }
        if (lane == 0) si[0] = bi;
    }
    __syncthreads();
    const int res = si[0];
    __syncthreads();
    return res;
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const float* __restrict__ top_p, const float* __restrict__ u, int* __restrict__ out,
              int V, size_t ld) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    __shared__ float sf[32];
    __shared__ int si[32];
    __shared__ float seg[THREADS];
    __shared__ int chosen;
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * ld;
    const float T = temperature ? temperature[r] : 0.f;
    if (!(T > 0.f)) {
        const int a = block_argmax(row, V, sf, si);
        if (threadIdx.x == 0) out[r] = a;
        return;
    }
    const float invT = 1.f / T;
    float mx = -INFINITY;
    for (int c = threadIdx.x; c < V; c += blockDim.x) mx = fmaxf(mx, row[c]);
    mx = bw::block_max(mx, sf);
    // contiguous segment of indices per thread: the CDF runs in index order
    const int per = (V + blockDim.x - 1) / blockDim.x;
    const int c0 = min(V, (int)threadIdx.x * per), c1 = min(V, c0 + per);

    float tau = 0.f;
    const float tp = top_p ? top_p[r] : 1.f;
    if (tp < 1.f) {
        float tot = 0.f;
        for (int c = c0; c < c1; ++c) tot += expf((row[c] - mx) * invT);
        tot = bw::block_sum(tot, sf);
        const float target = tp * tot;
        // largest float threshold whose kept mass still reaches the target (bisection on bits)
        unsigned lo = 0u, hi = __float_as_uint(1.0f) + 1u;  // mass(lo) >= target > mass(hi)
        while (hi - lo > 1u) {
            const unsigned mid = lo + ((hi - lo) >> 1);
            const float th = __uint_as_float(mid);
            float ms = 0.f;
            for (int c = c0; c < c1; ++c) { const float e = expf((row[c] - mx) * invT); if (e >= th) ms += e; }
            ms = bw::block_sum(ms, sf);
            if (ms >= target) lo = mid; else hi = mid;
        }
        tau = __uint_as_float(lo);
    }
    float mine = 0.f;
    for (int c = c0; c < c1; ++c) { const float e = expf((row[c] - mx) * invT); if (e >= tau) mine += e; }
    seg[threadIdx.x] = mine;
    if (threadIdx.x == 0) chosen = -1;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.f;
        for (int i = 0; i < (int)blockDim.x; ++i) tot += seg[i];
        const float goal = u[r] * tot;
        float run = 0.f; int owner = 0; bool found = false;
        for (int i = 0; i < (int)blockDim.x && !found; ++i) {
            if (seg[i] > 0.f) {
                owner = i;
                if (run + seg[i] > goal) found = true; else run += seg[i];
            }
        }
        if (!found) run -= seg[owner];  // goal at the very end: fall into the last kept segment
        // walk the owner's segment
        const int o0 = min(V, owner * per), o1 = min(V, o0 + per);
        int pick = -1, last = -1;
        for (int c = o0; c < o1; ++c) {
            const float e = expf((row[c] - mx) * invT);
            if (e >= tau) { last = c; run += e; if (run > goal) { pick = c; break; } }
        }
        chosen = pick >= 0 ? pick : last;
    }
    __syncthreads();
    if (threadIdx.x == 0) out[r] = chosen;
}

// Repetition penalty in place, one block per row: every DISTINCT id of the row's history
// ids[begin[r] .. begin[r+1]) has its logit divided by penalty[r] when positive and multiplied
// by it when not, once however often the id occurs (only an id's first occurrence acts).
// penalty <= 1 and ids outside [0, V) do nothing.
__global__ void repetition_penalty_kernel(float* __restrict__ logits, const int* __restrict__ ids,
                                          const int* __restrict__ begin, const float* __restrict__ penalty,
                                          int V, size_t ld) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    const int r = blockIdx.x;
    const float pen = penalty[r];
    if (!(pen > 1.f)) return;
    const int* mine = ids + begin[r];
    const int n = begin[r + 1] - begin[r];
    float* row = logits + (size_t)r * ld;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int id = mine[i];
        if (id < 0 || id >= V) continue;
        bool first = true;
        for (int j = 0; j < i && first; ++j) first = mine[j] != id;
        if (!first) continue;
        const float v = row[id];
        row[id] = v > 0.f ? v / pen : v * pen;
    }
}

// log softmax(row)[target[r]] per row, float32: (x_t - max) - log(sum exp(x - max)).
__global__ void __launch_bounds__(THREADS)
log_prob_kernel(const float* __restrict__ logits, const int* __restrict__ target, float* __restrict__ out,
                int V, size_t ld) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    __shared__ float sf[32];
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * ld;
    float mx = -INFINITY;
    for (int c = threadIdx.x; c < V; c += blockDim.x) mx = fmaxf(mx, row[c]);
    mx = bw::block_max(mx, sf);
    float s = 0.f;
    for (int c = threadIdx.x; c < V; c += blockDim.x) s += expf(row[c] - mx);
    s = bw::block_sum(s, sf);
    if (threadIdx.x == 0) out[r] = (row[target[r]] - mx) - logf(s);
}

}  // namespace

BW_EXPORT int bw_repetition_penalty(float* logits, const int* ids, const int* begin, const float* penalty,
                                    int R, int V, long long ld, void* stream) {
    if (R <= 0) return 0;
    if (V <= 0 || ld < V || !ids || !begin || !penalty) return BW_ERR_BAD_ARG;
    bw::launch((repetition_penalty_kernel), dim3(R), dim3(256), 0, (cudaStream_t)stream, logits, ids, begin, penalty,
               V, (size_t)ld);
    BW_LAUNCH_CHECK();
    return 0;
}

// target[r] must lie in [0, V): the caller checks it on the host.
BW_EXPORT int bw_log_prob(const float* logits, const int* target, float* out, int R, int V, long long ld,
                          void* stream) {
    if (R <= 0) return 0;
    if (V <= 0 || ld < V || !target || !out) return BW_ERR_BAD_ARG;
    bw::launch((log_prob_kernel), dim3(R), dim3(THREADS), 0, (cudaStream_t)stream, logits, target, out, V, (size_t)ld);
    BW_LAUNCH_CHECK();
    return 0;
}

// temperature, top_p: per row (may be null: greedy / no nucleus); u: per row uniform in [0,1).
BW_EXPORT int bw_sample(const float* logits, const float* temperature, const float* top_p, const float* u,
                        int* out, int R, int V, long long ld, void* stream) {
    if (R <= 0) return 0;
    if (V <= 0 || ld < V) return BW_ERR_BAD_ARG;
    if (temperature && !u) return BW_ERR_BAD_ARG;
    bw::launch((sample_kernel), dim3(R), dim3(THREADS), 0, (cudaStream_t)stream, logits, temperature, top_p, u, out, V, (size_t)ld);
    BW_LAUNCH_CHECK();
    return 0;
}
