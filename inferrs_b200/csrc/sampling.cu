// Token choice on the device, over float logits [rows, vocab].
//
// ib_argmax: greedy choice; among equal maxima the lowest token id wins.
#include "common.cuh"

__global__ void argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab, long ld) {
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const float* row = logits + (long)blockIdx.x * ld;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int j = threadIdx.x; j < vocab; j += blockDim.x) {
        const float v = row[j];
        if (v > bv || (v == bv && j < bi) || bi == 0x7fffffff) {
            if (!(v != v)) { bv = v; bi = j; }  // NaN never wins
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nwarps = (blockDim.x + 31) >> 5;
        bv = lane < nwarps ? best_v[lane] : -INFINITY;
        bi = lane < nwarps ? best_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
    }
}

IB_EXPORT int ib_argmax(const float* logits, int* out, int n_rows, int vocab, long ld, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (vocab <= 0) return IB_ERR_ARGUMENT;
    const int threads = vocab >= 8192 ? 1024 : 256;
    argmax_kernel<<<n_rows, threads, 0, stream>>>(logits, out, vocab, ld);
    return ib_launch_status();
}
