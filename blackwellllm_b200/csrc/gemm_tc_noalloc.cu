// The allocation-free variant of the split-K tensor-core matrix product; see
// gemm_tc_noalloc.h for who needs it and for its rules.  The kernels are those of
// gemm_tc.cu, compiled into this library as well; only the home of the split-K
// partial sums differs: a static device array instead of a caller's workspace.
#include "gemm_tc.cu"
#include "gemm_tc_noalloc.h"

// Scratch for the partial sums.  In host code this name is only a handle for the
// runtime (it is not a device address): the address comes from
// cudaGetSymbolAddress below and is what the kernels receive.
static __device__ __align__(256) float g_noalloc_scratch[BW_NOALLOC_SCRATCH_FLOATS];
// Completion counters of the split-K tiles.  They must be zero when a call starts: static device
// memory starts as zero, and the kernel sets every counter it used back to zero before it ends.
static __device__ __align__(256) int g_noalloc_counters[BW_NOALLOC_COUNTERS];

namespace {
constexpr int MAX_DEVICES = 64;
float* g_scratch_addr[MAX_DEVICES] = {nullptr};
int* g_counters_addr[MAX_DEVICES] = {nullptr};

// Device addresses of the scratch arrays on the current device; looked up once per device.
int scratch_on_current_device(float** addr, int** counters) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return BW_ERR_BAD_ARG;
    if (!g_scratch_addr[dev]) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        if (!p) return BW_ERR_DRIVER;
        int* c = nullptr;
        e = cudaGetSymbolAddress((void**)&c, g_noalloc_counters);
        if (e != cudaSuccess) return (int)e;
        if (!c) return BW_ERR_DRIVER;
        g_counters_addr[dev] = c;
        g_scratch_addr[dev] = p;
    }
    *addr = g_scratch_addr[dev];
    *counters = g_counters_addr[dev];
    return 0;
}
}  // namespace

BW_EXPORT int bw_gemm_tc_noalloc(const void* x, const void* w, const void* bias, int bias_type, void* out,
                                 int out_type, int M, int N, int K, long long ldx, long long ldo, int accumulate,
                                 int splits, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || splits < 1) return BW_ERR_BAD_ARG;
    const int kb_total = (K + BK - 1) / BK;
    if (splits > kb_total) splits = kb_total;
    if (splits > 1) {
        // only a product that is really split touches the arrays: its partial sums and one counter
        // group per output tile must fit them (an unsplit product of any size goes through)
        if ((long long)splits * M * N > (long long)BW_NOALLOC_SCRATCH_FLOATS) return BW_NOALLOC_TOO_LARGE;
        int tr = 0, bn = 0;
        bw_gemm_tc_plan(M, N, K, 0, 0, 0, &tr, &bn);
        const long long tiles = tr ? (long long)ceil_div(N, BM) * ceil_div(M, bn) : (long long)ceil_div(M, BM) * ceil_div(N, bn);
        if (tiles * 4 > (long long)BW_NOALLOC_COUNTERS) return BW_NOALLOC_TOO_LARGE;
    }
    float* scratch = nullptr;
    int* counters = nullptr;
    const int rc = scratch_on_current_device(&scratch, &counters);
    if (rc) return rc;
    return bw_gemm_tc(x, w, bias, bias_type, out, out_type, M, N, K, ldx, ldo, accumulate, /*swiglu=*/0, scratch,
                      (long long)BW_NOALLOC_SCRATCH_FLOATS, counters, (long long)BW_NOALLOC_COUNTERS, splits, stream);
}
