// Test-only kernel: one thread waits, through the package's bounded wait (bw::mbar_wait of
// csrc/tcgen05.cuh), for a barrier phase that nothing ever completes.  Built with a short limit
// (-DBW_WAIT_NS=2000000 -DBW_SPIN_LIMIT=4096), the wait gives up after about 2 ms, records its code
// in the status word and returns false; the kernel then ends normally.  Nothing faults and nothing
// waits forever: this is the path a broken pipeline would take in the real kernels.
#include "tcgen05.cuh"

__global__ void wait_probe_kernel(int* status, int* result, unsigned long long* waited_ns) {
    __shared__ __align__(8) uint64_t bar;
    const uint32_t b = bw::smem_u32(&bar);
    if (threadIdx.x == 0) {
        bw::mbar_init(b, 1);
        bw::fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint64_t t0 = bw::global_timer_ns();
        const bool ok = bw::mbar_wait(b, 0, status, 77);     // nobody arrives
        *waited_ns = bw::global_timer_ns() - t0;
        result[0] = ok ? 1 : 0;
        bw::mbar_arrive(b);                                   // now the phase completes ...
        result[1] = bw::mbar_wait(b, 0, status, 78) ? 1 : 0;  // ... and the same wait returns true at once
    }
}

BW_EXPORT int bw_wait_probe(int* status, int* result, unsigned long long* waited_ns, void* stream) {
    wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, result, waited_ns);
    BW_LAUNCH_CHECK();
    return 0;
}
