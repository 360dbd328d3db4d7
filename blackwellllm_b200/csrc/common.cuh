// Shared helpers for the sm_100a kernels of this engine.
//
// Every launcher is an extern "C" function over raw device pointers and a stream,
// returns 0 on success or a negative BW_ERR_* / positive cudaError_t code, and
// never allocates.  Python binds them with ctypes (kernels/ops.py).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define BW_EXPORT extern "C" __attribute__((visibility("default")))

// error codes returned by launchers (negative: ours; positive: cudaError_t)
#define BW_ERR_BAD_ARG   (-1)
#define BW_ERR_UNSUPPORTED (-2)
#define BW_ERR_DRIVER    (-3)

// element type codes used across the C interface
#define BW_F32  0
#define BW_BF16 1

// Programmatic dependent launch: a kernel launched through bw::launch may start while the kernel
// before it in the stream is still draining.  Such a kernel calls BW_PDL_TRIGGER() early (the next
// kernel may start launching) and BW_PDL_WAIT() before its first access to memory that an earlier
// kernel may write (everything but weights); the wait returns once all earlier kernels are
// complete and their writes visible.  Both are no-ops for ordinary launches.  BW_PDL=0 in the
// environment turns the early launch off.
#define BW_PDL_TRIGGER() asm volatile("griddepcontrol.launch_dependents;" ::: "memory")
#define BW_PDL_WAIT() asm volatile("griddepcontrol.wait;" ::: "memory")

#define BW_LAUNCH_CHECK() do { cudaError_t e__ = cudaGetLastError(); if (e__ != cudaSuccess) return (int)e__; } while (0)

#include <stdlib.h>
#include <utility>

namespace bw {

inline bool pdl_enabled() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("BW_PDL"); v = (e && e[0] == '0') ? 0 : 1; }
    return v != 0;
}

// overlap == false: an ordinary launch (the kernel starts when everything before it is complete)
template <typename... KArgs, typename... Args>
inline cudaError_t launch_opt(bool overlap, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = (overlap && pdl_enabled()) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// the same for a kernel whose CTAs come in clusters of two (grid.x even)
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pairs(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// The current device's number (0 where none can be asked: host-only use of a planner) and its number of SMs
// (148, the B200's, where none can be asked), looked up once per device.
constexpr int MAX_DEVICES = 64;
inline int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) { cudaGetLastError(); return 0; }
    return dev;
}
inline int num_sms() {
    static int cached[MAX_DEVICES] = {0};
    const int dev = current_device();
    if (cached[dev] <= 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) { cudaGetLastError(); n = 148; }
        cached[dev] = n;
    }
    return cached[dev];
}
// Raises a kernel's dynamic shared-memory limit once per device (`done`: one flag per device, zero-initialised).
template <typename K>
inline cudaError_t allow_dynamic_smem(K kernel, int bytes, bool (&done)[MAX_DEVICES]) {
    const int dev = current_device();
    if (done[dev]) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) done[dev] = true;
    return e;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          Args&&... args) {
    return launch_opt(true, kernel, grid, block, smem, stream, std::forward<Args>(args)...);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);   // lo in the low half
    return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum in a fixed order (lane tree, then warp 0 over the warp sums), so
// the result for a row never depends on which other rows are in the launch.
// `scratch` holds at least 32 floats.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : 0.f;
    r = warp_sum(r);
    return r;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}

}  // namespace bw
