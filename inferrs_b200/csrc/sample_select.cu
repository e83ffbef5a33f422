// Temperature / top-k / top-p / min-p sampling of one token per row, on the device.
//
// The order of operations is the reference sampler's (inferrs/src/sampler.rs:185-336):
// logits / T, softmax, sort by probability (descending, equal ones by token id), keep the
// first top_k, cut after the element whose cumulative probability reaches top_p, keep
// p >= min_p * p_max, renormalise, walk the kept list until the cumulative probability
// passes the random number u.  No list is sorted here.  With e_i = exp(z_i - z_max) every
// question the walk asks ("how much mass lies before rank r", "which rank holds mass t")
// is answered by a radix descent over the bits of e_i: four passes of 256 buckets, each
// bucket holding a count and a mass.  Masses are 64-bit integers (e * 2^40), so sums do
// not depend on the order of additions and a row's token does not depend on the batch.
//
// One block per row.  Rows with temperature < 1e-5 take the largest logit.
#include "common.cuh"

#define SMP_THREADS 1024
#define SMP_FIXED 1099511627776.0f  // 2^40

typedef unsigned long long u64;

__device__ __noinline__ float smp_elem(float logit, float temperature, float zmax) {
    const float z = logit / temperature;
    if (!(z == z)) return 0.0f;
    return expf(z - zmax);
}

__device__ __forceinline__ u64 smp_fixed(float e) { return __float2ull_rz(e * SMP_FIXED); }

__device__ __forceinline__ u64 smp_block_sum_u64(u64 v, u64* sh /* 32 */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    u64 r = lane < (blockDim.x >> 5) ? sh[lane] : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    return r;
}

struct SmpShared {
    unsigned int cnt[256];
    u64 mass[256];
    u64 red[32];
    float fred[32];
    int ired[32];
    // result of a descent step, written by thread 0
    int found;
    int bucket;
    unsigned int cnt_above;
    u64 mass_above;
    unsigned int c_tau;
    int scan[SMP_THREADS];
};

enum { SMP_COUNT_GE = 0, SMP_MASS_GE = 1, SMP_MASS_GT = 2 };

// Walk the sorted order (descending e) until the condition holds:
//   COUNT_GE: rank + 1 >= goal;  MASS_GE: mass up to and including the element >= goal;  MASS_GT: > goal.
// Returns the element's key `tau`, the count and mass of elements with key > tau, and how many share tau.
// found == 0: the condition never holds (the goal exceeds the totals).
__device__ void smp_descend(const float* __restrict__ row, int vocab, float temperature, float zmax, int mode,
                            u64 goal, SmpShared* sh, unsigned int* tau_out, unsigned int* cnt_above_out,
                            u64* mass_above_out, unsigned int* c_tau_out, int* found_out) {
    unsigned int prefix = 0, prefix_mask = 0;
    unsigned int cnt_above = 0;
    u64 mass_above = 0;
    unsigned int c_tau = 0;
    int found = 1;
    for (int level = 0; level < 4 && found; ++level) {
        const int shift = 24 - 8 * level;
        for (int b = threadIdx.x; b < 256; b += blockDim.x) { sh->cnt[b] = 0; sh->mass[b] = 0; }
        __syncthreads();
        int cur = -1;
        unsigned int cur_cnt = 0;
        u64 cur_mass = 0;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float e = smp_elem(row[i], temperature, zmax);
            const unsigned int key = __float_as_uint(e);
            if ((key & prefix_mask) != prefix) continue;
            const int b = (key >> shift) & 255;
            if (b != cur) {
                if (cur >= 0) { atomicAdd(&sh->cnt[cur], cur_cnt); atomicAdd(&sh->mass[cur], cur_mass); }
                cur = b; cur_cnt = 0; cur_mass = 0;
            }
            cur_cnt += 1;
            cur_mass += smp_fixed(e);
        }
        if (cur >= 0) { atomicAdd(&sh->cnt[cur], cur_cnt); atomicAdd(&sh->mass[cur], cur_mass); }
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned int c = cnt_above;
            u64 m = mass_above;
            int hit = -1;
            for (int b = 255; b >= 0; --b) {
                const unsigned int cb = sh->cnt[b];
                if (cb == 0) continue;
                const u64 mb = sh->mass[b];
                bool ok;
                if (mode == SMP_COUNT_GE) ok = (u64)c + cb >= goal;
                else if (mode == SMP_MASS_GE) ok = m + mb >= goal;
                else ok = m + mb > goal;
                if (ok) { hit = b; break; }
                c += cb;
                m += mb;
            }
            sh->found = hit >= 0;
            sh->bucket = hit;
            sh->cnt_above = c;
            sh->mass_above = m;
            sh->c_tau = hit >= 0 ? sh->cnt[hit] : 0;
        }
        __syncthreads();
        found = sh->found;
        if (found) {
            prefix |= ((unsigned int)sh->bucket) << shift;
            prefix_mask |= 255u << shift;
            cnt_above = sh->cnt_above;
            mass_above = sh->mass_above;
            c_tau = sh->c_tau;
        }
        __syncthreads();
    }
    *tau_out = prefix;
    *cnt_above_out = cnt_above;
    *mass_above_out = mass_above;
    *c_tau_out = c_tau;
    *found_out = found;
}

__global__ void __launch_bounds__(SMP_THREADS) sample_kernel(
    const float* __restrict__ logits, long ld, int vocab, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
    const float* __restrict__ uniform, int* __restrict__ out) {
    __shared__ SmpShared sh;
    ib_grid_dependency_sync();
    const int r = blockIdx.x;
    const float* row = logits + (long)r * ld;
    const float T = temperature[r];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    // largest logit and its lowest index (greedy answer, and z_max for the softmax)
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (v == v && (v > bv || bi == 0x7fffffff)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { sh.fred[warp] = bv; sh.ired[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = lane < (blockDim.x >> 5) ? sh.fred[lane] : -INFINITY;
        bi = lane < (blockDim.x >> 5) ? sh.ired[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) { sh.fred[0] = bv; sh.ired[0] = bi == 0x7fffffff ? 0 : bi; }
    }
    __syncthreads();
    const float lmax = sh.fred[0];
    const int imax = sh.ired[0];
    __syncthreads();
    if (T < 1e-5f || !(lmax > -INFINITY)) {
        if (threadIdx.x == 0) out[r] = imax;
        return;
    }
    const float zmax = lmax / T;

    // total mass
    u64 part = 0;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) part += smp_fixed(smp_elem(row[i], T, zmax));
    const u64 total = smp_block_sum_u64(part, sh.red);

    unsigned int keep_cnt = vocab;
    u64 keep_mass = total;
    unsigned int tau, ca, ct;
    u64 ma;
    int found;
    const int k = top_k[r];
    if (k > 0 && k < vocab) {
        smp_descend(row, vocab, T, zmax, SMP_COUNT_GE, (u64)k, &sh, &tau, &ca, &ma, &ct, &found);
        if (found) {
            keep_cnt = k;
            keep_mass = ma + (u64)(k - ca) * smp_fixed(__uint_as_float(tau));
        }
    }
    const float tp = top_p[r];
    if (tp < 1.0f) {
        const u64 goal = (u64)((double)tp * (double)total);
        smp_descend(row, vocab, T, zmax, SMP_MASS_GE, goal, &sh, &tau, &ca, &ma, &ct, &found);
        if (found) {
            const u64 pm = smp_fixed(__uint_as_float(tau));
            u64 n = 1;
            if (pm > 0 && goal > ma) n = (goal - ma + pm - 1) / pm;
            if (n < 1) n = 1;
            if (n > ct) n = ct;
            if (ca + n < keep_cnt) { keep_cnt = ca + (unsigned int)n; keep_mass = ma + n * pm; }
        }
    }
    const float mp = min_p[r];
    if (mp > 0.0f) {
        // e_max is 1, so "p >= min_p * p_max" is "e >= min_p"
        unsigned int c = 0;
        u64 m = 0;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float e = smp_elem(row[i], T, zmax);
            if (e >= mp) { c += 1; m += smp_fixed(e); }
        }
        const u64 cm = smp_block_sum_u64((u64)c, sh.red);
        const u64 mm = smp_block_sum_u64(m, sh.red);
        if (cm > 0 && cm < keep_cnt) { keep_cnt = (unsigned int)cm; keep_mass = mm; }
    }

    // the element of the kept list whose interval of cumulative mass holds u * keep_mass
    u64 target = (u64)((double)uniform[r] * (double)keep_mass);
    if (keep_mass > 0 && target >= keep_mass) target = keep_mass - 1;
    smp_descend(row, vocab, T, zmax, SMP_MASS_GT, target, &sh, &tau, &ca, &ma, &ct, &found);
    if (!found) {  // no mass at all: the most probable token
        if (threadIdx.x == 0) out[r] = imax;
        return;
    }
    const u64 pm = smp_fixed(__uint_as_float(tau));
    u64 n = pm > 0 ? (target - ma) / pm : 0;
    if (n >= ct) n = ct - 1;
    if (ca + n >= keep_cnt) n = keep_cnt > ca ? keep_cnt - 1 - ca : 0;

    // the n-th token, in order of token id, whose key is tau
    const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
    const int i0 = threadIdx.x * chunk, i1 = min(vocab, i0 + chunk);
    int mine = 0;
    for (int i = i0; i < i1; ++i) mine += (__float_as_uint(smp_elem(row[i], T, zmax)) == tau);
    sh.scan[threadIdx.x] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int t = 0; t < blockDim.x; ++t) { const int c = sh.scan[t]; sh.scan[t] = run; run += c; }
    }
    __syncthreads();
    const int before = sh.scan[threadIdx.x];
    if ((u64)before <= n && n < (u64)before + mine) {
        int seen = before;
        for (int i = i0; i < i1; ++i) {
            if (__float_as_uint(smp_elem(row[i], T, zmax)) == tau) {
                if ((u64)seen == n) { out[r] = i; break; }
                ++seen;
            }
        }
    }
}

IB_EXPORT int ib_sample(const float* logits, long ld, int n_rows, int vocab, const float* temperature,
                        const int* top_k, const float* top_p, const float* min_p, const float* uniform, int* out,
                        cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (vocab <= 0) return IB_ERR_ARGUMENT;
    sample_kernel<<<n_rows, SMP_THREADS, 0, stream>>>(logits, ld, vocab, temperature, top_k, top_p, min_p, uniform,
                                                      out);
    return ib_launch_status();
}
