// See decode_step.h.  Host code only (compiled by nvcc for its CUDA runtime).
#include <cuda_runtime.h>
#include <vector>
#include "decode_step.h"

#define BW_EXPORT extern "C" __attribute__((visibility("default")))

namespace {
typedef long long (*PackFn)(void*, int, int*, const int*, const int*, const int*, const int*, int, int, long long, int*,
                            long long, long long*, int*);
typedef long long (*LengthFn)(void*, int);
typedef int (*TruncateFn)(void*, int, long long);
typedef int (*SampleFn)(const float*, const float*, const float*, const float*, int*, int, int, long long, void*);
PackFn g_pack = nullptr;
LengthFn g_length = nullptr;
TruncateFn g_truncate = nullptr;
SampleFn g_sample = nullptr;
// the host runtime's codes (host_runtime.cpp)
constexpr long long BWH_NO_SLOT = -1, BWH_OUT_OF_PAGES = -2;
}  // namespace

BW_EXPORT int bw_decode_step_bind(void* pack_step, void* length, void* truncate, void* sample) {
    if (!pack_step || !length || !truncate || !sample) return BW_STEP_INVALID_ARGUMENT;
    g_pack = (PackFn)pack_step; g_length = (LengthFn)length; g_truncate = (TruncateFn)truncate; g_sample = (SampleFn)sample;
    return BW_STEP_SUCCESS;
}

BW_EXPORT int bw_decode_step(bw_decode_step_args* a) {
    if (!g_pack) return BW_STEP_STATE_MISMATCH;
    if (!a || a->n <= 0 || !a->cache || !a->handles || !a->tokens || !a->positions || !a->pinned || !a->device_step ||
        !a->graph_exec || !a->logits || !a->sampled_device)
        return BW_STEP_INVALID_ARGUMENT;
    a->cuda_error = 0;
    const int n = a->n;
    // positions against the cache: equal = decode on, lower = rewind first, higher = a gap
    for (int i = 0; i < n; ++i) {
        const long long len = g_length(a->cache, a->handles[i]);
        if (len < 0) return BW_STEP_STATE_MISMATCH;
        if (a->positions[i] > len) return BW_STEP_STATE_MISMATCH;
        if (a->positions[i] < 0 || a->positions[i] >= a->max_context) return BW_STEP_INVALID_ARGUMENT;
    }
    for (int i = 0; i < n; ++i)
        if (a->positions[i] < g_length(a->cache, a->handles[i]) && g_truncate(a->cache, a->handles[i], a->positions[i]) != 0)
            return BW_STEP_STATE_MISMATCH;
    static thread_local std::vector<int> ones, zeros, new_slots;
    if ((int)ones.size() < n) { ones.assign(n, 1); zeros.assign(n, 0); new_slots.assign(n, 0); }
    long long meta[4 + 16] = {0};
    const long long total = g_pack(a->cache, n, a->handles, ones.data(), a->tokens, ones.data(), zeros.data(), a->vocab,
                                   a->table_width, 1LL << 40, a->pinned, a->pinned_words, meta, new_slots.data());
    if (total == BWH_OUT_OF_PAGES || total == BWH_NO_SLOT) return BW_STEP_OUT_OF_PAGES;
    if (total < 0) return BW_STEP_INVALID_ARGUMENT;
    if (total != a->step_words) {
        // a sequence outgrew the context the graph was captured for: take the growth back
        for (int i = 0; i < n; ++i) g_truncate(a->cache, a->handles[i], a->positions[i]);
        return BW_STEP_INVALID_CONFIG;
    }
    cudaStream_t s = (cudaStream_t)a->stream;
    cudaError_t e = cudaMemcpyAsync(a->device_step, a->pinned, (size_t)total * sizeof(int), cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess && a->device_tokens)
        e = cudaMemcpyAsync(a->device_step, a->device_tokens, (size_t)n * sizeof(int), cudaMemcpyDeviceToDevice, s);
    if (e == cudaSuccess) e = cudaGraphLaunch((cudaGraphExec_t)a->graph_exec, s);
    if (e != cudaSuccess) {
        for (int i = 0; i < n; ++i) g_truncate(a->cache, a->handles[i], a->positions[i]);
        a->cuda_error = (int)e;
        return BW_STEP_CUDA_RUNTIME_ERROR;
    }
    const int rc = g_sample(a->logits, nullptr, nullptr, nullptr, a->sampled_device, n, a->vocab, a->logits_ld, a->stream);
    if (rc != 0) { a->cuda_error = rc; return BW_STEP_CUDA_RUNTIME_ERROR; }
    if (a->sampled_host) {
        e = cudaMemcpyAsync(a->sampled_host, a->sampled_device, (size_t)n * sizeof(int), cudaMemcpyDeviceToHost, s);
        if (e == cudaSuccess && a->wait) e = cudaStreamSynchronize(s);
        if (e != cudaSuccess) { a->cuda_error = (int)e; return BW_STEP_CUDA_RUNTIME_ERROR; }
    }
    return BW_STEP_SUCCESS;
}
