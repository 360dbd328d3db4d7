// Memory-bound row kernels: embedding gather, RMSNorm (optionally on gathered rows),
// SwiGLU, and rotary position encoding fused with the append of keys and values
// into cache pages.  All arithmetic is 32-bit; inputs and outputs are float32 or
// bfloat16 as the type codes say.  Any width is accepted (no power-of-two rule).
#include "common.cuh"

using bf16 = __nv_bfloat16;

namespace {

// ---------------------------------------------------------------- embedding
template <typename WT>
__global__ void embed_gather_kernel(const WT* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int H, int V, float scale) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= V) id = 0;  // the host rejects such ids before the launch
    const WT* row = table + (size_t)id * H;
    float* o = out + (size_t)t * H;
    const int c0 = blockIdx.y * blockDim.x * 4;   // each block copies 4 * blockDim elements of the row
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int c = c0 + k * blockDim.x + threadIdx.x;
        if (c < H) o[c] = bw::to_f32(row[c]) * scale;   // scale 1: the stored value
    }
}

// ---------------------------------------------------------------- RMSNorm
// y = x * rsqrt(mean(x^2) + eps) * w.  One block per output row; input row is
// rows[i] when `rows` is given (final norm on the rows whose logits are wanted).
template <typename WT, typename OT>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const WT* __restrict__ w,
                               const int* __restrict__ rows, OT* __restrict__ out,
                               int H, float eps) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    __shared__ float scratch[32];
    const int i = blockIdx.x;
    const int src = rows ? rows[i] : i;
    const float* xr = x + (size_t)src * H;
    OT* o = out + (size_t)i * H;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) { float v = xr[c]; ss = fmaf(v, v, ss); }
    ss = bw::block_sum(ss, scratch);
    const float r = rsqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x)
        o[c] = bw::from_f32<OT>(xr[c] * r * bw::to_f32(w[c]));
}

// The same with 4 elements per access, for widths that are multiples of 4 (the sum runs over
// the same per-thread strided order scaled by 4; rows stay independent of one another).
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&r.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 r;
    r.x = *reinterpret_cast<uint32_t*>(&a); r.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = r;
}

template <typename WT, typename OT>
__global__ void rmsnorm_vec4_kernel(const float* __restrict__ x, const WT* __restrict__ w,
                                    const int* __restrict__ rows, OT* __restrict__ out, int H, float eps) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    __shared__ float scratch[32];
    const int i = blockIdx.x;
    const int src = rows ? rows[i] : i;
    const float* xr = x + (size_t)src * H;
    OT* o = out + (size_t)i * H;
    float ss = 0.f;
    for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
        const float4 v = load4(xr + c);
        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
    ss = bw::block_sum(ss, scratch);
    const float r = rsqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
        const float4 v = load4(xr + c), g = load4(w + c);
        store4(o + c, make_float4(v.x * r * g.x, v.y * r * g.y, v.z * r * g.z, v.w * r * g.w));
    }
}

// v += p[0] + p[stride] + ... (n values, added in that order; four loads in flight at a time)
__device__ __forceinline__ void add_planes4(float4& v, const float* p, int n, size_t stride) {
    for (int p0 = 0; p0 < n; p0 += 4) {
        float4 t[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) t[j] = p0 + j < n ? load4(p + (size_t)(p0 + j) * stride) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 4; ++j) { v.x += t[j].x; v.y += t[j].y; v.z += t[j].z; v.w += t[j].w; }
    }
}
__device__ __forceinline__ void add_planes1(float& v, const float* p, int n, size_t stride) {
    for (int p0 = 0; p0 < n; p0 += 4) {
        float t[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) t[j] = p0 + j < n ? p[(size_t)(p0 + j) * stride] : 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) v += t[j];
    }
}

// x += planes[0] + planes[1] + ... (in that order), then the norm of the new x: the planes are a matrix
// product that its kernel left unsummed (bw_gemm_tc_planes).  One block per output row.  With
// `rows` (the final norm on chosen rows, which may repeat) x is left as it is and only the norm's
// input is the sum.  Every thread re-reads only what it wrote itself.
template <typename WT, typename OT, bool VEC>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ planes, int n_planes,
                                   size_t plane_stride, const WT* __restrict__ w, const int* __restrict__ rows,
                                   OT* __restrict__ out, int H, float eps) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    __shared__ float scratch[32];
    const int i = blockIdx.x;
    const int src = rows ? rows[i] : i;
    float* xr = x + (size_t)src * H;
    const float* pr = planes + (size_t)src * H;
    OT* o = out + (size_t)i * H;
    constexpr int W = VEC ? 4 : 1;
    float ss = 0.f;
    for (int c = threadIdx.x * W; c < H; c += blockDim.x * W) {
        if constexpr (VEC) {
            float4 v = load4(xr + c);
            add_planes4(v, pr + c, n_planes, plane_stride);
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
            if (!rows) store4(xr + c, v);
        } else {
            float v = xr[c];
            add_planes1(v, pr + c, n_planes, plane_stride);
            ss = fmaf(v, v, ss);
            if (!rows) xr[c] = v;
        }
    }
    ss = bw::block_sum(ss, scratch);
    const float r = rsqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x * W; c < H; c += blockDim.x * W) {
        if constexpr (VEC) {
            float4 v = load4(xr + c);
            if (rows) add_planes4(v, pr + c, n_planes, plane_stride);
            const float4 g = load4(w + c);
            store4(o + c, make_float4(v.x * r * g.x, v.y * r * g.y, v.z * r * g.z, v.w * r * g.w));
        } else {
            float v = xr[c];
            if (rows) add_planes1(v, pr + c, n_planes, plane_stride);
            o[c] = bw::from_f32<OT>(v * r * bw::to_f32(w[c]));
        }
    }
}

// x += planes[0] + planes[1] + ... (in that order)
__global__ void add_planes_kernel(float* __restrict__ x, const float* __restrict__ planes, int n_planes,
                                  size_t plane_stride, size_t total) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float v = x[i];
        add_planes1(v, planes + i, n_planes, plane_stride);
        x[i] = v;
    }
}

// ---------------------------------------------------------------- SwiGLU
// in: [T, 2I] with gate in columns [0, I) and up in [I, 2I); out: [T, I].
template <typename IT, typename OT>
__global__ void swiglu_kernel(const IT* __restrict__ gu, OT* __restrict__ out, int I, size_t total) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I; const int c = (int)(idx - t * I);
        const float g = bw::to_f32(gu[t * 2 * (size_t)I + c]);
        const float u = bw::to_f32(gu[t * 2 * (size_t)I + I + c]);
        const float s = g / (1.f + expf(-g));
        out[idx] = bw::from_f32<OT>(s * u);
    }
}

// ---------------------------------------------------------------- RoPE + append
// qkv: [T, (nh + 2 nkv) * hd] (q heads, then k heads, then v heads).
// q_out: [T, nh * hd] rotated queries.  Rotated keys and raw values go to the
// page of the token's position: pages are [num_pages, nkv, page_size, hd].
// rotary_dim = 0 rotates nothing (a mixer without rotary encoding).
// cos and sin of pos * inv_freq[j] for every token of the step: [T, rotary_dim] (cos, then sin).
// All layers with the same rotary parameters share one table per step.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float* __restrict__ table, int rotary_dim, int T) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    const int half = rotary_dim >> 1;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * half) return;
    const int t = idx / half, j = idx - t * half;
    float s, c;
    sincosf((float)positions[t] * inv_freq[j], &s, &c);
    table[(size_t)t * rotary_dim + j] = c;
    table[(size_t)t * rotary_dim + half + j] = s;
}

// Where each token of the step keeps its keys and values: page * page_size + slot of its position,
// or -1 when the block table names no page there.  The same for all layers of a cache group.
__global__ void kv_slots_kernel(const int* __restrict__ positions, const int* __restrict__ req_of_token,
                                const int* __restrict__ block_table, int max_blocks, int page_size, int num_pages,
                                int* __restrict__ kv_slot, int T) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    const int pos = positions[t];
    const int page = block_table[(size_t)req_of_token[t] * max_blocks + pos / page_size];
    kv_slot[t] = (page >= 0 && page < num_pages) ? page * page_size + pos % page_size : -1;
}

constexpr int ROPE_HPB = 8;   // heads per block of rope_append_kernel

template <typename IT, typename OT>
__global__ void rope_append_kernel(const IT* __restrict__ qkv, const int* __restrict__ positions,
                                   const int* __restrict__ req_of_token,
                                   const int* __restrict__ block_table, int max_blocks,
                                   const float* __restrict__ inv_freq, const float* __restrict__ table,
                                   int rotary_dim, OT* __restrict__ q_out, OT* __restrict__ k_pages,
                                   OT* __restrict__ v_pages, int nh, int nkv, int hd,
                                   int page_size, int num_pages, int paired, int n_planes, size_t plane_stride) {
    BW_PDL_TRIGGER();
    // A block takes ROPE_HPB heads of one token; a thread takes one channel of each of them: the
    // loads of the heads are independent and in flight together, the angle is looked up once.
    // Positions and block tables were on the device before the step's first kernel ran, so the page
    // is looked up before the wait for the kernels that make qkv and the table.
    const int t = blockIdx.x, h0 = blockIdx.y * ROPE_HPB;
    const int n_heads = nh + 2 * nkv;
    const int pos = positions[t];
    const int half = rotary_dim >> 1;
    const IT* row = qkv + (size_t)t * n_heads * hd;
    int page = -1, slot = 0;
    if (h0 + ROPE_HPB > nh) {   // this block holds key or value heads
        const int r = req_of_token[t];
        page = block_table[(size_t)r * max_blocks + pos / page_size];
        slot = pos % page_size;
        if (page >= num_pages) page = -1;
    }
    BW_PDL_WAIT();
    for (int c = threadIdx.x; c < hd; c += blockDim.x) {
        float sn = 0.f, cs = 1.f;
        const bool rot_c = c < rotary_dim;
        if (rot_c) {
            const int j = c < half ? c : c - half;
            if (table) { cs = table[(size_t)t * rotary_dim + j]; sn = table[(size_t)t * rotary_dim + half + j]; }
            else sincosf((float)pos * inv_freq[j], &sn, &cs);
            if (c < half) sn = -sn;   // first half: x cos - partner sin; second half: partner sin + x cos
        }
        // paired: in the q and k heads the input holds channel j and its partner j + half side by side
        // (at 2j and 2j + 1), the order the fused projection's weight rows have
        const int sc = (paired && rot_c) ? (c < half ? 2 * c : 2 * (c - half) + 1) : c;
        const int pc = rot_c ? (paired ? (sc ^ 1) : (c < half ? c + half : c - half)) : c;
        float v[ROPE_HPB], w[ROPE_HPB];
#pragma unroll
        for (int k = 0; k < ROPE_HPB; ++k) {
            const int h = h0 + k;
            v[k] = h < n_heads ? bw::to_f32(row[(size_t)h * hd + (h < nh + nkv ? sc : c)]) : 0.f;
            w[k] = (h < nh + nkv && rot_c) ? bw::to_f32(row[(size_t)h * hd + pc]) : 0.f;
        }
        // qkv left as planes by its matrix product: the further planes are added in order
        for (int p0 = 1; p0 < n_planes; p0 += 2) {   // two planes' loads in flight together
            float tv[2][ROPE_HPB], tw[2][ROPE_HPB];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const IT* prow = row + (size_t)(p0 + j) * plane_stride;
                const bool there = p0 + j < n_planes;
#pragma unroll
                for (int k = 0; k < ROPE_HPB; ++k) {
                    const int h = h0 + k;
                    tv[j][k] = (there && h < n_heads) ? bw::to_f32(prow[(size_t)h * hd + (h < nh + nkv ? sc : c)]) : 0.f;
                    tw[j][k] = (there && h < nh + nkv && rot_c) ? bw::to_f32(prow[(size_t)h * hd + pc]) : 0.f;
                }
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
#pragma unroll
                for (int k = 0; k < ROPE_HPB; ++k) { v[k] += tv[j][k]; w[k] += tw[j][k]; }
            }
        }
#pragma unroll
        for (int k = 0; k < ROPE_HPB; ++k) {
            const int h = h0 + k;
            if (h >= n_heads) break;
            const float o = (h < nh + nkv && rot_c) ? v[k] * cs + w[k] * sn : v[k];
            if (h < nh) {
                q_out[((size_t)t * nh + h) * hd + c] = bw::from_f32<OT>(o);
            } else if (page >= 0) {
                const bool is_k = h < nh + nkv;
                const int kvh = is_k ? h - nh : h - nh - nkv;
                (is_k ? k_pages : v_pages)[(((size_t)page * nkv + kvh) * page_size + slot) * hd + c] = bw::from_f32<OT>(o);
            }
        }
    }
}

// ---------------------------------------------------------------- logits
// In place: x * scale, then cap * tanh(x / cap) when cap > 0 (a model's logit multiplier and soft cap).
__global__ void logit_transform_kernel(float* __restrict__ x, long long n, float scale, float cap) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float v = x[i] * scale;
        if (cap > 0.f) v = cap * tanhf(v * inv_cap);
        x[i] = v;
    }
}

template <typename T> const T* cp(const void* p) { return reinterpret_cast<const T*>(p); }
template <typename T> T* mp(void* p) { return reinterpret_cast<T*>(p); }

}  // namespace

BW_EXPORT int bw_logit_transform(float* logits, long long n, float scale, float cap, void* stream) {
    if (n <= 0) return 0;
    const int threads = 256;
    const long long blocks = (n + threads - 1) / threads;
    bw::launch(logit_transform_kernel, dim3((unsigned)(blocks < 148 * 16 ? blocks : 148 * 16)), dim3(threads), 0,
               (cudaStream_t)stream, logits, n, scale, cap);
    BW_LAUNCH_CHECK();
    return 0;
}

BW_EXPORT int bw_embed_gather(const void* table, int table_type, const int* ids, float* out,
                              int T, int H, int V, float scale, void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = H >= 1024 ? 256 : 128;
    const dim3 grid(T, (H + threads * 4 - 1) / (threads * 4));
    if (table_type == BW_F32) bw::launch((embed_gather_kernel<float>), dim3(grid), dim3(threads), 0, s, cp<float>(table), ids, out, H, V, scale);
    else if (table_type == BW_BF16) bw::launch((embed_gather_kernel<bf16>), dim3(grid), dim3(threads), 0, s, cp<bf16>(table), ids, out, H, V, scale);
    else return BW_ERR_BAD_ARG;
    BW_LAUNCH_CHECK();
    return 0;
}

BW_EXPORT int bw_rmsnorm(const float* x, const void* w, int w_type, const int* rows, void* out,
                         int out_type, int n_rows, int H, float eps, void* stream) {
    if (n_rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = H % 4 == 0 && (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) == 0;
    const int threads = vec ? (H >= 4096 ? 512 : (H >= 1024 ? 256 : 128)) : (H >= 2048 ? 512 : (H >= 512 ? 256 : 128));
#define BW_RMS(WT, OT) do { if (vec) bw::launch((rmsnorm_vec4_kernel<WT, OT>), dim3(n_rows), dim3(threads), 0, s, x, cp<WT>(w), rows, mp<OT>(out), H, eps); \
        else bw::launch((rmsnorm_kernel<WT, OT>), dim3(n_rows), dim3(threads), 0, s, x, cp<WT>(w), rows, mp<OT>(out), H, eps); } while (0)
    if (w_type == BW_F32 && out_type == BW_F32) BW_RMS(float, float);
    else if (w_type == BW_F32 && out_type == BW_BF16) BW_RMS(float, bf16);
    else if (w_type == BW_BF16 && out_type == BW_F32) BW_RMS(bf16, float);
    else if (w_type == BW_BF16 && out_type == BW_BF16) BW_RMS(bf16, bf16);
    else return BW_ERR_BAD_ARG;
#undef BW_RMS
    BW_LAUNCH_CHECK();
    return 0;
}

// x[n_rows or more, H] += the planes (float32, plane_stride floats apart), out = rmsnorm of the new x.
// rows != null: out row i is the norm of x[rows[i]] + planes[.][rows[i]], and x is NOT changed.
BW_EXPORT int bw_add_rmsnorm(float* x, const float* planes, int n_planes, long long plane_stride, const void* w,
                             int w_type, const int* rows, void* out, int out_type, int n_rows, int H, float eps,
                             void* stream) {
    if (n_rows <= 0) return 0;
    if (!planes || n_planes < 1 || plane_stride < 0) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = H % 4 == 0 && plane_stride % 4 == 0 &&
                     (((uintptr_t)x | (uintptr_t)planes | (uintptr_t)w | (uintptr_t)out) & 15) == 0;
    // one pass over the row: a thread per four elements (up to 1,024 threads), so that the loads of
    // the stream and of all planes are in flight at once
    const int quads = (H / 4 + 31) / 32 * 32;
    const int threads = vec ? (quads > 1024 ? 1024 : (quads < 128 ? 128 : quads)) : (H >= 2048 ? 512 : (H >= 512 ? 256 : 128));
#define BW_ARMS(WT, OT) do { if (vec) bw::launch((add_rmsnorm_kernel<WT, OT, true>), dim3(n_rows), dim3(threads), 0, s, x, planes, n_planes, (size_t)plane_stride, cp<WT>(w), rows, mp<OT>(out), H, eps); \
        else bw::launch((add_rmsnorm_kernel<WT, OT, false>), dim3(n_rows), dim3(threads), 0, s, x, planes, n_planes, (size_t)plane_stride, cp<WT>(w), rows, mp<OT>(out), H, eps); } while (0)
    if (w_type == BW_F32 && out_type == BW_F32) BW_ARMS(float, float);
    else if (w_type == BW_F32 && out_type == BW_BF16) BW_ARMS(float, bf16);
    else if (w_type == BW_BF16 && out_type == BW_F32) BW_ARMS(bf16, float);
    else if (w_type == BW_BF16 && out_type == BW_BF16) BW_ARMS(bf16, bf16);
    else return BW_ERR_BAD_ARG;
#undef BW_ARMS
    BW_LAUNCH_CHECK();
    return 0;
}

// x[total] += the planes, added in plane order
BW_EXPORT int bw_add_planes(float* x, const float* planes, int n_planes, long long plane_stride, long long total,
                            void* stream) {
    if (total <= 0 || n_planes <= 0) return 0;
    if (!x || !planes || plane_stride < 0) return BW_ERR_BAD_ARG;
    const long long want = (total + 255) / 256;
    bw::launch(add_planes_kernel, dim3((unsigned)(want < 148 * 8 ? want : 148 * 8)), dim3(256), 0, (cudaStream_t)stream,
               x, planes, n_planes, (size_t)plane_stride, (size_t)total);
    BW_LAUNCH_CHECK();
    return 0;
}

BW_EXPORT int bw_swiglu(const void* gu, int in_type, void* out, int out_type, int T, int I, void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)T * I;
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
    if (in_type == BW_F32 && out_type == BW_F32) bw::launch((swiglu_kernel<float, float>), dim3(blocks), dim3(threads), 0, s, cp<float>(gu), mp<float>(out), I, total);
    else if (in_type == BW_BF16 && out_type == BW_BF16) bw::launch((swiglu_kernel<bf16, bf16>), dim3(blocks), dim3(threads), 0, s, cp<bf16>(gu), mp<bf16>(out), I, total);
    else if (in_type == BW_F32 && out_type == BW_BF16) bw::launch((swiglu_kernel<float, bf16>), dim3(blocks), dim3(threads), 0, s, cp<float>(gu), mp<bf16>(out), I, total);
    else return BW_ERR_BAD_ARG;
    BW_LAUNCH_CHECK();
    return 0;
}

BW_EXPORT int bw_rope_table(const int* positions, const float* inv_freq, float* table, int rotary_dim, int T,
                            void* stream) {
    if (T <= 0 || rotary_dim <= 0) return 0;
    if (rotary_dim & 1) return BW_ERR_BAD_ARG;
    const int total = T * (rotary_dim / 2);
    bw::launch((rope_table_kernel), dim3((total + 255) / 256), dim3(256), 0, (cudaStream_t)stream, positions, inv_freq, table, rotary_dim, T);
    BW_LAUNCH_CHECK();
    return 0;
}

BW_EXPORT int bw_kv_slots(const int* positions, const int* req_of_token, const int* block_table, int max_blocks,
                          int page_size, int num_pages, int* kv_slot, int T, void* stream) {
    if (T <= 0) return 0;
    if (page_size <= 0 || (long long)num_pages * page_size > 2147483647LL) return BW_ERR_BAD_ARG;
    bw::launch((kv_slots_kernel), dim3((T + 127) / 128), dim3(128), 0, (cudaStream_t)stream, positions, req_of_token,
               block_table, max_blocks, page_size, num_pages, kv_slot, T);
    BW_LAUNCH_CHECK();
    return 0;
}

// table: [T, rotary_dim] from bw_rope_table, or null to compute the angles here.  paired != 0: the
// rotated channels of the q and k heads come as (channel j, channel j + rotary_dim / 2) pairs.
// n_planes > 1: qkv is the sum of that many planes, plane_stride elements apart (bw_gemm_tc_planes).
BW_EXPORT int bw_rope_append(const void* qkv, int in_type, const int* positions, const int* req_of_token,
                             const int* block_table, int max_blocks, const float* inv_freq, const float* table,
                             int rotary_dim, void* q_out, void* k_pages, void* v_pages, int out_type,
                             int T, int nh, int nkv, int hd, int page_size, int num_pages, int paired,
                             int n_planes, long long plane_stride, void* stream) {
    if (T <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > hd || (rotary_dim & 1) || n_planes < 1 || (n_planes > 1 && plane_stride <= 0)) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = hd >= 256 ? 256 : (hd >= 128 ? 128 : (hd >= 64 ? 64 : 32));
    const dim3 grid(T, (nh + 2 * nkv + ROPE_HPB - 1) / ROPE_HPB);
#define BW_RA(IT, OT) bw::launch((rope_append_kernel<IT, OT>), dim3(grid), dim3(threads), 0, s, cp<IT>(qkv), positions, req_of_token, \
        block_table, max_blocks, inv_freq, table, rotary_dim, mp<OT>(q_out), mp<OT>(k_pages), mp<OT>(v_pages), \
        nh, nkv, hd, page_size, num_pages, paired, n_planes, (size_t)plane_stride)
    if (in_type == BW_F32 && out_type == BW_F32) BW_RA(float, float);
    else if (in_type == BW_F32 && out_type == BW_BF16) BW_RA(float, bf16);
    else if (in_type == BW_BF16 && out_type == BW_BF16) BW_RA(bf16, bf16);
    else return BW_ERR_BAD_ARG;
#undef BW_RA
    BW_LAUNCH_CHECK();
    return 0;
}
