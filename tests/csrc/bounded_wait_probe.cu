// Test-only: the bounded mbarrier wait of the package's kernels (sm100.cuh) on a barrier that nobody arrives at,
// with a limit of a millisecond or so.  No copy is in flight and nothing spins beyond the limit: the kernel
// returns, reports through the status words, and the context stays usable.
#include <cuda_runtime.h>

#include "sm100.cuh"

using namespace sm100;

// status[0]: 1 the wait completed, 0 it ran out; status[1]: microseconds the wait took
__global__ void bounded_wait_probe_kernel(int* status, int* error_word, unsigned long long limit_ns, int arrive) {
    __shared__ unsigned long long bar;
    const unsigned b = smem_u32(&bar);
    if (threadIdx.x == 0) {
        mbar_init(b, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (arrive && threadIdx.x == 1) mbar_arrive(b);
    if (threadIdx.x == 0) {
        const unsigned long long t0 = global_ns();
        const bool ok = mbar_wait_bounded(b, 0, error_word, 7, limit_ns);
        status[0] = ok ? 1 : 0;
        status[1] = (int)((global_ns() - t0) / 1000ull);
    }
}

extern "C" __attribute__((visibility("default"))) int bounded_wait_probe(int* status, int* error_word,
                                                                        unsigned long long limit_ns, int arrive,
                                                                        cudaStream_t stream) {
    bounded_wait_probe_kernel<<<1, 32, 0, stream>>>(status, error_word, limit_ns, arrive);
    return (int)cudaPeekAtLastError();
}
