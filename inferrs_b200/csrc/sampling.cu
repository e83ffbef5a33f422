// Token choice on the device, over float logits [rows, vocab].
//
// ib_argmax: greedy choice; among equal maxima the lowest token id wins.
#include "common.cuh"

__global__ void argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab, long ld) {
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    ib_grid_dependency_sync();
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

// Two-stage form for few rows: the vocabulary is cut into chunks, one block each, so that a single row still
// fills the machine.  A partial result is one 64-bit word, (ordered value bits << 32) | ~index, whose
// unsigned maximum is the largest value and, among equal values, the lowest index.
#define ARGMAX_CHUNK 8192

__device__ __forceinline__ unsigned long long argmax_pack(float v, int i) {
    unsigned b = __float_as_uint(v);
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);  // unsigned order = float order
    return ((unsigned long long)b << 32) | (unsigned long long)(0xffffffffu - (unsigned)i);
}

__global__ void argmax_partial_kernel(const float* __restrict__ logits, unsigned long long* __restrict__ part,
                                      int vocab, long ld, int n_chunks) {
    __shared__ unsigned long long red[32];
    ib_grid_dependency_sync();
    const float* row = logits + (long)blockIdx.x * ld;
    const int j0 = blockIdx.y * ARGMAX_CHUNK;
    const int j1 = j0 + ARGMAX_CHUNK < vocab ? j0 + ARGMAX_CHUNK : vocab;
    unsigned long long best = 0;  // below every packed value of a real number
    for (int j = j0 + threadIdx.x; j < j1; j += blockDim.x) {
        const float v = row[j];
        if (v == v) {
            const unsigned long long p = argmax_pack(v, j);
            best = p > best ? p : best;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x < 32) {
        best = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
            best = other > best ? other : best;
        }
        if (threadIdx.x == 0) part[(long)blockIdx.x * n_chunks + blockIdx.y] = best;
    }
}

__global__ void argmax_final_kernel(const unsigned long long* __restrict__ part, int* __restrict__ out, int n_chunks) {
    ib_grid_dependency_sync();
    unsigned long long best = 0;
    for (int c = threadIdx.x; c < n_chunks; c += 32) {
        const unsigned long long p = part[(long)blockIdx.x * n_chunks + c];
        best = p > best ? p : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    if (threadIdx.x == 0) out[blockIdx.x] = best == 0 ? 0 : (int)(0xffffffffu - (unsigned)(best & 0xffffffffu));
}

// scratch: n_rows * ceil(vocab / 8192) 64-bit words, or nullptr for the one-block-per-row form
IB_EXPORT int ib_argmax(const float* logits, int* out, int n_rows, int vocab, long ld, void* scratch,
                        cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (vocab <= 0) return IB_ERR_ARGUMENT;
    const int n_chunks = (vocab + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK;
    if (scratch != nullptr && n_chunks > 1) {
        ib_launch(argmax_partial_kernel, dim3(n_rows, n_chunks), 512, 0, stream, logits, (unsigned long long*)scratch, vocab,
                  ld, n_chunks);
        ib_launch(argmax_final_kernel, n_rows, 32, 0, stream, (const unsigned long long*)scratch, out, n_chunks);
        return ib_launch_status();
    }
    const int threads = vocab >= 8192 ? 1024 : 256;
    ib_launch(argmax_kernel, n_rows, threads, 0, stream, logits, out, vocab, ld);
    return ib_launch_status();
}

// ---------------------------------------------------------------------------
// Penalties on the logits of tokens seen lately (in place, before sampling):
//   repetition: logit / p if logit >= 0 else logit * p, once per distinct token;
//   frequency:  logit -= f * (times seen);  presence: logit -= q  (seen at least once).
// prev [rows, max_prev] holds each row's window of previous tokens, n_prev[row] of them valid.
// ---------------------------------------------------------------------------
__global__ void penalties_kernel(float* __restrict__ logits, long ld, int vocab, const int* __restrict__ prev,
                                 int max_prev, const int* __restrict__ n_prev, const float* __restrict__ repetition,
                                 const float* __restrict__ frequency, const float* __restrict__ presence) {
    ib_grid_dependency_sync();
    const int row = blockIdx.x;
    const int n = n_prev[row] < max_prev ? n_prev[row] : max_prev;
    const float rp = repetition[row], fp = frequency[row], pp = presence[row];
    const bool use_rp = rp != 1.0f && rp != 0.0f;
    const bool use_fp = fp != 0.0f || pp != 0.0f;
    if (n <= 0 || (!use_rp && !use_fp)) return;
    const int* p = prev + (long)row * max_prev;
    float* l = logits + (long)row * ld;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int id = p[i];
        if (id < 0 || id >= vocab) continue;
        bool first = true;
        for (int j = 0; j < i; ++j)
            if (p[j] == id) { first = false; break; }
        if (!first) continue;  // the first occurrence's thread updates the logit: no two threads share one
        int count = 1;
        for (int j = i + 1; j < n; ++j) count += (p[j] == id);
        float v = l[id];
        if (use_rp) v = v >= 0.0f ? v / rp : v * rp;
        if (use_fp) { v -= fp * (float)count; v -= pp; }
        l[id] = v;
    }
}

IB_EXPORT int ib_penalties(float* logits, long ld, int n_rows, int vocab, const int* prev, int max_prev,
                           const int* n_prev, const float* repetition, const float* frequency,
                           const float* presence, cudaStream_t stream) {
    if (n_rows <= 0 || max_prev <= 0) return IB_OK;
    penalties_kernel<<<n_rows, 256, 0, stream>>>(logits, ld, vocab, prev, max_prev, n_prev, repetition, frequency,
                                                  presence);
    return ib_launch_status();
}
