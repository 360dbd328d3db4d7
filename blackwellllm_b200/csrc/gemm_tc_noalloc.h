// bw_gemm_tc_noalloc: the split-K tensor-core matrix product for callers that must
// not allocate device memory.
//
// This entry point has no counterpart in the reference project (fxslava/BlackwellLLM);
// it exists for this library's own users.
//
// Who needs it: code that runs where cudaMalloc is off limits -- inside a stream
// capture (an allocation there is either an error or ends the capture), in a
// latency-critical loop whose owner has handed out all device memory up front, or
// in a host process that embeds this library under a fixed memory budget and
// forbids every allocating call, torch's caching allocator included.  The regular
// entry point (bw_gemm_tc) needs the caller to bring a float32 workspace for the
// split-K partial sums; this one brings its own.
//
// How: the partial sums live in a file-scope `static __device__` array inside the
// library, BW_NOALLOC_SCRATCH_FLOATS floats (16 MiB).  Every GPU on which the
// library is loaded holds that array until the process exits.  The call makes no
// cudaMalloc, cudaFree or other allocating call.
//
// Limits and rules:
//   * With more than one split (after the clamp to the number of 64-wide
//     k-blocks), splits * M * N must not exceed BW_NOALLOC_SCRATCH_FLOATS and the
//     product must not have more than BW_NOALLOC_COUNTERS / 4 output tiles (of
//     128 features x up to 16..256 tokens), else the call returns
//     BW_NOALLOC_TOO_LARGE (-10) and launches nothing.  A product with one split
//     uses neither array and is not bounded by them.
//   * The first call on a device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current) and keeps it.  Make that
//     first call before any stream capture begins.
//   * All calls on a device share the one array.  Two calls that overlap on the
//     GPU (different streams, no dependency between them) race on it and give
//     wrong sums; order them on one stream or with events.
//   * The array keeps the last call's contents.  The partial sums need no
//     clearing: every one a call reads was written by that same call.  Beside
//     them sit BW_NOALLOC_COUNTERS int32 completion counters (64 KiB) that must be
//     zero when a call starts; they start as zero and every call puts the ones it
//     used back to zero before its kernel ends.
//   * Operands as for bw_gemm_tc: x [M, K] and w [N, K] bfloat16 with K and ldx
//     multiples of 8 and 16-byte aligned bases; out [M, N] float32 or bfloat16
//     (type codes 0 / 1), accumulate != 0 adds into a float32 out.
#pragma once

#define BW_NOALLOC_SCRATCH_FLOATS (4 * 1024 * 1024)
#define BW_NOALLOC_COUNTERS 16384
#define BW_NOALLOC_TOO_LARGE (-10)

#ifdef __cplusplus
extern "C" {
#endif

// out[M, N] (=|+=) x[M, K] . w[N, K]^T (+ bias[N]), K cut into `splits` parts (>= 1;
// clamped to the number of 64-wide k-blocks) whose float32 partial sums are added in
// split order.  Returns 0, BW_NOALLOC_TOO_LARGE, another negative BW_ERR_* code, or
// a positive cudaError_t.
int bw_gemm_tc_noalloc(const void* x, const void* w, const void* bias, int bias_type, void* out, int out_type,
                       int M, int N, int K, long long ldx, long long ldo, int accumulate, int splits,
                       void* stream);

#ifdef __cplusplus
}
#endif
