// Temperature / top-k / top-p / min-p sampling of one token per row, on the device.
//
// The order of operations is the reference sampler's (inferrs/src/sampler.rs:185-336):
// logits / T, softmax, sort by probability (descending, equal ones by token id), keep the
// first top_k, cut after the element whose cumulative probability reaches top_p, keep
// p >= min_p * p_max, renormalise, walk the kept list until the cumulative probability
// passes the random number u.  No list is sorted here.  With e_i = exp(z_i - z_max) every
// question the walk asks ("how much mass lies before rank r", "which rank holds mass t")
// is answered by a radix descent over the bits of e_i: four levels of 256 buckets, each
// bucket holding a count and a mass.  Masses are 64-bit integers (e * 2^40), so sums do
// not depend on the order of additions and a row's token does not depend on the batch.
//
// How the work is laid out (a vocabulary of 150,000 and a handful of rows would otherwise
// keep a handful of SMs busy for milliseconds):
//   * a row is taken by a cluster of 1, 2, 4 or 8 CTAs, each with its own stretch of the
//     vocabulary; after every pass each CTA adds up all CTAs' bucket tables through
//     distributed shared memory and comes to the same decision as the others;
//   * e_i is computed once, in the pass that also fills the first level's table, and kept in a
//     float32 scratch row; that table serves all descents (top-k, top-p, the final walk), and
//     the later levels only look at the scratch row's bits;
//   * a warp adds its 32 elements to a table of its own: lanes that share a bucket are found
//     with a ballot and summed with a warp reduction, so that atomic operations are left for
//     lanes whose bucket no other lane has.
//   * with top-k on, what can still be chosen after it (the elements above the k-th and all that
//     share its key: the head of the sorted order) is gathered into shared memory once, and the
//     top-p cut, min-p, the draw and the look-up of the drawn token go over that list.
#include "common.cuh"

#define SMP_THREADS 1024
#define SMP_WARPS (SMP_THREADS / 32)
#define SMP_FIXED 1099511627776.0f  // 2^40
#define SMP_MAX_CLUSTER 8
#define SMP_LIST 2048                  // most elements that the list after top-k may hold (over all CTAs of a row)
#define SMP_UNROLL 4                   // loads that a thread has on their way in the passes over a row

typedef unsigned long long u64;

__device__ __forceinline__ float smp_elem(float logit, float temperature, float zmax) {
    const float z = logit / temperature;
    if (!(z == z)) return 0.0f;
    return expf(z - zmax);
}

__device__ __forceinline__ u64 smp_fixed(float e) { return __float2ull_rz(e * SMP_FIXED); }

// ---- the cluster -------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned smp_cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ unsigned smp_cluster_size() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void smp_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
template <typename T>
__device__ __forceinline__ T smp_remote(const T* local, unsigned rank) {   // the same variable in another CTA of the cluster
    const unsigned addr = (unsigned)__cvta_generic_to_shared(local);
    unsigned remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    T v;
    if constexpr (sizeof(T) == 8) {
        unsigned long long raw;
        asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(raw) : "r"(remote) : "memory");
        v = *reinterpret_cast<T*>(&raw);
    } else {
        unsigned raw;
        asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(raw) : "r"(remote) : "memory");
        v = *reinterpret_cast<T*>(&raw);
    }
    return v;
}

// What a CTA shows the others of its cluster: two copies, used in turn, so that one cluster barrier per exchange is
// enough (a CTA may fill the next copy while a slower one still reads the last).
struct SmpBoard {
    unsigned int cnt[256];
    u64 mass[256];
    u64 sums[2];        // two numbers of a plain sum (min-p's count and mass; the matches of the last scan)
    float best;         // largest logit of this CTA's stretch, and its lowest index
    int best_at;
};

struct SmpShared {
    SmpBoard board[2];
    unsigned int cnt0[256];   // the first level's table of the whole row
    u64 mass0[256];
    unsigned int cnt[256];    // the table of the whole row after the last pass
    u64 mass[256];
    u64 red[32];
    float fred[32];
    int ired[32];
    int scan[SMP_THREADS];
    // the elements that survive top-k (those with a key above the k-th's, and all that share it): the head of the
    // sorted order, as far as this CTA's stretch holds it
    unsigned int list_key[SMP_LIST];
    int list_at[SMP_LIST];
    int list_n;
    // a descent step's answer, written by thread 0
    int found, bucket;
    unsigned int cnt_above, c_tau;
    u64 mass_above;
};

struct SmpCtx {
    SmpShared* sh;
    unsigned int* warp_cnt;   // [SMP_WARPS][256], dynamic shared memory
    u64* warp_mass;           // [SMP_WARPS][256]
    unsigned rank, size;
    int turn;                 // which copy of the board the next exchange uses
    int lo, hi;               // this CTA's stretch of the vocabulary
};

// One element per lane into the warp's own table.  The lanes that share the first active lane's bucket (at the
// first level, where the buckets are e's exponents, often most of the warp; in a row of equal logits all of it, at
// every level) are found with a ballot and summed with a warp reduction; the others go in with shared-memory
// atomics, which then meet few lanes with the same bucket.  (Measured on 148 rows of random logits: 455 us with one
// such round, 477 with two, 678 with as many as there are buckets, 425 with none; on 148 rows of equal logits 716 us
// with one round and 4,005 with none.)
__device__ __forceinline__ void smp_warp_add(unsigned int* wc, u64* wm, bool active, int bucket, u64 mass) {
    const int lane = threadIdx.x & 31;
    const unsigned todo = __ballot_sync(0xffffffffu, active);
    if (todo) {
        const int leader = __ffs(todo) - 1;
        const int lb = __shfl_sync(0xffffffffu, bucket, leader);
        const bool mine = active && bucket == lb;
        const unsigned grp = __ballot_sync(0xffffffffu, mine);
        // a mass is below 2^41: twenty low bits and twenty-one high bits, each summed over 32 lanes in 32 bits
        const unsigned lo = __reduce_add_sync(0xffffffffu, mine ? (unsigned)(mass & 0xFFFFFu) : 0u);
        const unsigned hi = __reduce_add_sync(0xffffffffu, mine ? (unsigned)(mass >> 20) : 0u);
        if (lane == leader) {
            wc[lb] += (unsigned)__popc(grp);
            wm[lb] += ((u64)hi << 20) + lo;
        }
        active = active && !mine;
    }
    __syncwarp();   // the leader's plain additions are done before anybody's atomic ones, and before the next call
    if (active) {
        atomicAdd(&wc[bucket], 1u);
        atomicAdd(&wm[bucket], mass);
    }
    __syncwarp();
}

__device__ __forceinline__ void smp_clear_warp_tables(const SmpCtx& c) {
    for (int i = threadIdx.x; i < SMP_WARPS * 256; i += SMP_THREADS) { c.warp_cnt[i] = 0; c.warp_mass[i] = 0; }
    __syncthreads();
}

// the warps' tables -> this CTA's board -> the row's table in sh->cnt / sh->mass of every CTA of the cluster
__device__ void smp_merge_tables(SmpCtx& c) {
    SmpShared* sh = c.sh;
    __syncthreads();
    SmpBoard* board = &sh->board[c.turn];
    for (int b = threadIdx.x; b < 256; b += SMP_THREADS) {
        unsigned int n = 0;
        u64 m = 0;
        for (int w = 0; w < SMP_WARPS; ++w) { n += c.warp_cnt[w * 256 + b]; m += c.warp_mass[w * 256 + b]; }
        board->cnt[b] = n;
        board->mass[b] = m;
    }
    if (c.size > 1) smp_cluster_sync(); else __syncthreads();
    for (int b = threadIdx.x; b < 256; b += SMP_THREADS) {
        unsigned int n = 0;
        u64 m = 0;
        for (unsigned r = 0; r < c.size; ++r) {
            n += c.size > 1 ? smp_remote(&board->cnt[b], r) : board->cnt[b];
            m += c.size > 1 ? smp_remote(&board->mass[b], r) : board->mass[b];
        }
        sh->cnt[b] = n;
        sh->mass[b] = m;
    }
    c.turn ^= 1;
    __syncthreads();
}

// The same for a table that the threads have added to this CTA's board directly (the few elements of the list, with
// atomics): clear_board before, exchange_board after.
__device__ void smp_clear_board(SmpCtx& c) {
    SmpBoard* board = &c.sh->board[c.turn];
    for (int b = threadIdx.x; b < 256; b += SMP_THREADS) { board->cnt[b] = 0; board->mass[b] = 0; }
    __syncthreads();
}
__device__ void smp_exchange_board(SmpCtx& c) {
    SmpShared* sh = c.sh;
    SmpBoard* board = &sh->board[c.turn];
    if (c.size > 1) smp_cluster_sync(); else __syncthreads();
    for (int b = threadIdx.x; b < 256; b += SMP_THREADS) {
        unsigned int n = 0;
        u64 m = 0;
        for (unsigned r = 0; r < c.size; ++r) {
            n += c.size > 1 ? smp_remote(&board->cnt[b], r) : board->cnt[b];
            m += c.size > 1 ? smp_remote(&board->mass[b], r) : board->mass[b];
        }
        sh->cnt[b] = n;
        sh->mass[b] = m;
    }
    c.turn ^= 1;
    __syncthreads();
}

// two numbers summed over the block and then over the cluster; every thread gets both sums
__device__ void smp_sum2(SmpCtx& c, u64 a, u64 b, u64* a_out, u64* b_out) {
    SmpShared* sh = c.sh;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { a += __shfl_xor_sync(0xffffffffu, a, o); b += __shfl_xor_sync(0xffffffffu, b, o); }
    __syncthreads();
    if (lane == 0) sh->red[warp] = a;
    __syncthreads();
    u64 ta = 0;
    if (threadIdx.x == 0) for (int w = 0; w < SMP_WARPS; ++w) ta += sh->red[w];
    __syncthreads();
    if (lane == 0) sh->red[warp] = b;
    __syncthreads();
    SmpBoard* board = &sh->board[c.turn];
    if (threadIdx.x == 0) {
        u64 tb = 0;
        for (int w = 0; w < SMP_WARPS; ++w) tb += sh->red[w];
        board->sums[0] = ta;
        board->sums[1] = tb;
    }
    if (c.size > 1) smp_cluster_sync(); else __syncthreads();
    u64 sa = 0, sb = 0;
    for (unsigned r = 0; r < c.size; ++r) {
        sa += c.size > 1 ? smp_remote(&board->sums[0], r) : board->sums[0];
        sb += c.size > 1 ? smp_remote(&board->sums[1], r) : board->sums[1];
    }
    c.turn ^= 1;
    *a_out = sa;
    *b_out = sb;
    __syncthreads();
}

enum { SMP_COUNT_GE = 0, SMP_MASS_GE = 1, SMP_MASS_GT = 2 };

// Walk the sorted order (descending e) until the condition holds:
//   COUNT_GE: rank + 1 >= goal;  MASS_GE: mass up to and including the element >= goal;  MASS_GT: > goal.
// Returns the element's key `tau`, the count and mass of elements with key > tau, and how many share tau.
// found == 0: the condition never holds (the goal exceeds the totals).  The first level reads the table that the
// pass over the logits made; the others make theirs from the bits of the scratch row.
// With `from_list` the elements are those of the list in shared memory instead of the row's (the list is the head of
// the sorted order, so whatever holds at a rank inside it is found there as in the row), at every level.
__device__ void smp_descend(SmpCtx& c, const float* __restrict__ e_row, bool from_list, int mode, u64 goal,
                            unsigned int* tau_out, unsigned int* cnt_above_out, u64* mass_above_out,
                            unsigned int* c_tau_out, int* found_out) {
    SmpShared* sh = c.sh;
    unsigned int prefix = 0, prefix_mask = 0;
    unsigned int cnt_above = 0;
    u64 mass_above = 0;
    unsigned int c_tau = 0;
    int found = 1;
    for (int level = 0; level < 4 && found; ++level) {
        const int shift = 24 - 8 * level;
        const unsigned int* cnt = sh->cnt0;
        const u64* mass = sh->mass0;
        if (from_list) {
            smp_clear_board(c);
            SmpBoard* board = &sh->board[c.turn];
            for (int j = threadIdx.x; j < sh->list_n; j += SMP_THREADS) {
                const unsigned int key = sh->list_key[j];
                if ((key & prefix_mask) == prefix) {
                    atomicAdd(&board->cnt[(key >> shift) & 255], 1u);
                    atomicAdd(&board->mass[(key >> shift) & 255], smp_fixed(__uint_as_float(key)));
                }
            }
            smp_exchange_board(c);
            cnt = sh->cnt;
            mass = sh->mass;
        } else if (level > 0) {
            smp_clear_warp_tables(c);
            unsigned int* wc = c.warp_cnt + (threadIdx.x >> 5) * 256;
            u64* wm = c.warp_mass + (threadIdx.x >> 5) * 256;
            // the same number of rounds for every lane of a warp; four loads on their way per lane
            for (int i0 = c.lo; i0 < c.hi; i0 += SMP_UNROLL * SMP_THREADS) {
                float e[SMP_UNROLL];
#pragma unroll
                for (int u = 0; u < SMP_UNROLL; ++u) {
                    const int i = i0 + u * SMP_THREADS + threadIdx.x;
                    e[u] = i < c.hi ? e_row[i] : 0.0f;
                }
#pragma unroll
                for (int u = 0; u < SMP_UNROLL; ++u) {
                    const int i = i0 + u * SMP_THREADS + threadIdx.x;
                    const unsigned int key = __float_as_uint(e[u]);
                    const bool active = i < c.hi && (key & prefix_mask) == prefix;
                    if (__any_sync(0xffffffffu, active)) smp_warp_add(wc, wm, active, (key >> shift) & 255, smp_fixed(e[u]));
                }
            }
            smp_merge_tables(c);
            cnt = sh->cnt;
            mass = sh->mass;
        }
        if (threadIdx.x < 32) {
            // lane l looks at buckets 255 - 8 l down to 248 - 8 l; what lies before them comes from a scan over the lanes
            const int lane = threadIdx.x;
            unsigned int n_loc[8], n_sum = 0;
            u64 m_loc[8], m_sum = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int b = 255 - (8 * lane + j);
                n_loc[j] = cnt[b];
                m_loc[j] = mass[b];
                n_sum += n_loc[j];
                m_sum += m_loc[j];
            }
            unsigned int n_inc = n_sum;
            u64 m_inc = m_sum;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned int tn = __shfl_up_sync(0xffffffffu, n_inc, o);
                const u64 tm = __shfl_up_sync(0xffffffffu, m_inc, o);
                if (lane >= o) { n_inc += tn; m_inc += tm; }
            }
            unsigned int n = cnt_above + (n_inc - n_sum);
            u64 m = mass_above + (m_inc - m_sum);
            int hit = -1;
            unsigned int hit_cnt = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const unsigned int cb = n_loc[j];
                if (hit >= 0 || cb == 0) continue;
                bool ok;
                if (mode == SMP_COUNT_GE) ok = (u64)n + cb >= goal;
                else if (mode == SMP_MASS_GE) ok = m + m_loc[j] >= goal;
                else ok = m + m_loc[j] > goal;
                if (ok) { hit = 255 - (8 * lane + j); hit_cnt = cb; }
                else { n += cb; m += m_loc[j]; }
            }
            // the sums grow from lane to lane, so the first lane with a hit holds the first bucket with one
            const unsigned who = __ballot_sync(0xffffffffu, hit >= 0);
            if (who == 0) {
                if (lane == 0) { sh->found = 0; sh->bucket = -1; sh->c_tau = 0; }
            } else if (lane == __ffs(who) - 1) {
                sh->found = 1;
                sh->bucket = hit;
                sh->cnt_above = n;
                sh->mass_above = m;
                sh->c_tau = hit_cnt;
            }
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
    const float* __restrict__ uniform, float* __restrict__ scratch, int* __restrict__ out) {
    __shared__ SmpShared sh;
    extern __shared__ __align__(16) unsigned char smp_dynamic[];
    ib_grid_dependency_sync();
    SmpCtx c;
    c.sh = &sh;
    c.warp_mass = reinterpret_cast<u64*>(smp_dynamic);
    c.warp_cnt = reinterpret_cast<unsigned int*>(smp_dynamic + (size_t)SMP_WARPS * 256 * sizeof(u64));
    c.size = smp_cluster_size();
    c.rank = smp_cluster_rank();
    c.turn = 0;
    const int r = blockIdx.x / c.size;
    const int stretch = (vocab + (int)c.size - 1) / (int)c.size;
    c.lo = min(vocab, (int)c.rank * stretch);
    c.hi = min(vocab, c.lo + stretch);
    const float* row = logits + (long)r * ld;
    float* e_row = scratch + (long)r * vocab;
    const float T = temperature[r];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    // largest logit and its lowest index (greedy answer, and z_max for the softmax)
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = c.lo + threadIdx.x; i < c.hi; i += SMP_THREADS) {
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
        bv = lane < SMP_WARPS ? sh.fred[lane] : -INFINITY;
        bi = lane < SMP_WARPS ? sh.ired[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) { sh.board[c.turn].best = bv; sh.board[c.turn].best_at = bi; }
    }
    if (c.size > 1) smp_cluster_sync(); else __syncthreads();
    float lmax = -INFINITY;
    int imax = 0x7fffffff;
    for (unsigned k = 0; k < c.size; ++k) {   // the same answer in every CTA
        const float ov = c.size > 1 ? smp_remote(&sh.board[c.turn].best, k) : sh.board[c.turn].best;
        const int oi = c.size > 1 ? smp_remote(&sh.board[c.turn].best_at, k) : sh.board[c.turn].best_at;
        if (ov > lmax || (ov == lmax && oi < imax)) { lmax = ov; imax = oi; }
    }
    if (imax == 0x7fffffff) imax = 0;
    c.turn ^= 1;
    __syncthreads();
    if (T < 1e-5f || !(lmax > -INFINITY)) {
        if (threadIdx.x == 0 && c.rank == 0) out[r] = imax;
        // a CTA's board may still be read by the others: nobody leaves before everybody has read
        if (c.size > 1) smp_cluster_sync();
        return;
    }
    const float zmax = lmax / T;

    // e_i into the scratch row, and the first level's table (which holds the total mass too)
    smp_clear_warp_tables(c);
    {
        unsigned int* wc = c.warp_cnt + warp * 256;
        u64* wm = c.warp_mass + warp * 256;
        for (int i0 = c.lo; i0 < c.hi; i0 += SMP_UNROLL * SMP_THREADS) {
            float v[SMP_UNROLL];
#pragma unroll
            for (int u = 0; u < SMP_UNROLL; ++u) {
                const int i = i0 + u * SMP_THREADS + threadIdx.x;
                v[u] = i < c.hi ? row[i] : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < SMP_UNROLL; ++u) {
                const int i = i0 + u * SMP_THREADS + threadIdx.x;
                const bool active = i < c.hi;
                const float e = active ? smp_elem(v[u], T, zmax) : 0.0f;
                if (active) e_row[i] = e;
                smp_warp_add(wc, wm, active, (int)(__float_as_uint(e) >> 24), smp_fixed(e));
            }
        }
    }
    __syncthreads();   // this CTA's stretch of the scratch row is read by other threads from here on
    smp_merge_tables(c);
    u64 part = 0;
    for (int b = threadIdx.x; b < 256; b += SMP_THREADS) {
        sh.cnt0[b] = sh.cnt[b];
        sh.mass0[b] = sh.mass[b];
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        for (int b = threadIdx.x; b < 256; b += 32) part += sh.mass0[b];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        if (threadIdx.x == 0) sh.red[0] = part;
    }
    __syncthreads();
    const u64 total = sh.red[0];
    __syncthreads();

    unsigned int keep_cnt = vocab;
    u64 keep_mass = total;
    unsigned int tau, ca, ct;
    u64 ma;
    int found;
    // With top-k on, the elements that can still be chosen (those above the k-th, and all that share its key) are
    // few.  They are gathered into shared memory once; the top-p cut, min-p, the draw and the look-up of the drawn
    // token then go over this list, which is the head of the sorted order, instead of over the row.
    bool listed = false;
    const int k = top_k[r];
    if (k > 0 && k < vocab) {
        smp_descend(c, e_row, false, SMP_COUNT_GE, (u64)k, &tau, &ca, &ma, &ct, &found);
        if (found) {
            keep_cnt = k;
            keep_mass = ma + (u64)(k - ca) * smp_fixed(__uint_as_float(tau));
            if ((u64)ca + ct <= SMP_LIST) {
                if (threadIdx.x == 0) sh.list_n = 0;
                __syncthreads();
                for (int i0 = c.lo; i0 < c.hi; i0 += SMP_UNROLL * SMP_THREADS) {
                    float e[SMP_UNROLL];
#pragma unroll
                    for (int u = 0; u < SMP_UNROLL; ++u) {
                        const int i = i0 + u * SMP_THREADS + threadIdx.x;
                        e[u] = i < c.hi ? e_row[i] : 0.0f;
                    }
#pragma unroll
                    for (int u = 0; u < SMP_UNROLL; ++u) {
                        const int i = i0 + u * SMP_THREADS + threadIdx.x;
                        const unsigned int key = __float_as_uint(e[u]);   // e >= 0: the bits order as the values do
                        if (i < c.hi && key >= tau) {
                            const int at = atomicAdd(&sh.list_n, 1);
                            sh.list_key[at] = key;
                            sh.list_at[at] = i;
                        }
                    }
                }
                __syncthreads();
                listed = true;
            }
        }
    }
    const float tp = top_p[r];
    if (tp < 1.0f) {
        const u64 goal = (u64)((double)tp * (double)total);
        // with the list: a goal beyond the mass of the first k is reached behind them, where the cut changes nothing
        if (!listed || goal <= keep_mass) {
            smp_descend(c, e_row, listed, SMP_MASS_GE, goal, &tau, &ca, &ma, &ct, &found);
            if (found) {
                const u64 pm = smp_fixed(__uint_as_float(tau));
                u64 n = 1;
                if (pm > 0 && goal > ma) n = (goal - ma + pm - 1) / pm;
                if (n < 1) n = 1;
                if (n > ct) n = ct;
                if (ca + n < keep_cnt) { keep_cnt = ca + (unsigned int)n; keep_mass = ma + n * pm; }
            }
        }
    }
    const float mp = min_p[r];
    if (mp > 0.0f) {
        // e_max is 1, so "p >= min_p * p_max" is "e >= min_p".  Over the list the count is the row's whenever it is
        // below keep_cnt (then some listed element fails, and with it every element behind the list).
        u64 n = 0, m = 0;
        if (listed) {
            for (int j = threadIdx.x; j < sh.list_n; j += SMP_THREADS) {
                const float e = __uint_as_float(sh.list_key[j]);
                if (e >= mp) { n += 1; m += smp_fixed(e); }
            }
        } else {
            for (int i = c.lo + threadIdx.x; i < c.hi; i += SMP_THREADS) {
                const float e = e_row[i];
                if (e >= mp) { n += 1; m += smp_fixed(e); }
            }
        }
        u64 cm, mm;
        smp_sum2(c, n, m, &cm, &mm);
        if (cm > 0 && cm < keep_cnt) { keep_cnt = (unsigned int)cm; keep_mass = mm; }
    }

    // the element of the kept list whose interval of cumulative mass holds u * keep_mass
    u64 target = (u64)((double)uniform[r] * (double)keep_mass);
    if (keep_mass > 0 && target >= keep_mass) target = keep_mass - 1;
    smp_descend(c, e_row, listed, SMP_MASS_GT, target, &tau, &ca, &ma, &ct, &found);
    if (!found) {  // no mass at all: the most probable token
        if (threadIdx.x == 0 && c.rank == 0) out[r] = imax;
        if (c.size > 1) smp_cluster_sync();
        return;
    }
    const u64 pm = smp_fixed(__uint_as_float(tau));
    u64 n = pm > 0 ? (target - ma) / pm : 0;
    if (n >= ct) n = ct - 1;
    if (ca + n >= keep_cnt) n = keep_cnt > ca ? keep_cnt - 1 - ca : 0;

    // the n-th token, in order of token id, whose key is tau
    SmpBoard* board = &sh.board[c.turn];
    if (listed) {
        // this CTA's matches, and those of the CTAs with lower ranks (whose token ids are all lower)
        int mine = 0;
        for (int j = threadIdx.x; j < sh.list_n; j += SMP_THREADS) mine += (sh.list_key[j] == tau);
        mine = (int)ib_warp_sum((float)mine);           // at most 2,048: exact in float32
        if (lane == 0) sh.ired[warp] = mine;
        __syncthreads();
        if (threadIdx.x == 0) {
            int all = 0;
            for (int w = 0; w < SMP_WARPS; ++w) all += sh.ired[w];
            board->sums[0] = (u64)all;
        }
        if (c.size > 1) smp_cluster_sync(); else __syncthreads();
        u64 before = 0;
        for (unsigned k2 = 0; k2 < c.rank; ++k2) before += smp_remote(&board->sums[0], k2);
        for (int j = threadIdx.x; j < sh.list_n; j += SMP_THREADS) {
            if (sh.list_key[j] != tau) continue;
            const int at = sh.list_at[j];
            u64 place = before;                         // matches with a lower token id
            for (int j2 = 0; j2 < sh.list_n; ++j2) place += (sh.list_key[j2] == tau && sh.list_at[j2] < at);
            if (place == n) out[r] = at;
        }
        if (c.size > 1) smp_cluster_sync();   // nobody leaves while its board may still be read
        return;
    }
    // over the row: every thread counts a stretch of its own, the stretches before it (in its CTA, and in the CTAs
    // with lower ranks) tell it where its matches stand
    const int chunk = (c.hi - c.lo + SMP_THREADS - 1) / SMP_THREADS;
    const int i0 = min(c.hi, c.lo + (int)threadIdx.x * chunk), i1 = min(c.hi, i0 + chunk);
    int mine = 0;
    for (int i = i0; i < i1; ++i) mine += (__float_as_uint(e_row[i]) == tau);
    int upto = mine;                       // matches of this warp's lanes up to and including this one
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, upto, o);
        if (lane >= o) upto += t;
    }
    if (lane == 31) sh.ired[warp] = upto;
    __syncthreads();
    if (warp == 0) {                       // the warps' totals: each warp's start, and the CTA's total
        const int mine_w = lane < SMP_WARPS ? sh.ired[lane] : 0;
        int upto_w = mine_w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, upto_w, o);
            if (lane >= o) upto_w += t;
        }
        sh.scan[lane] = upto_w - mine_w;
        if (lane == 31) board->sums[0] = (u64)upto_w;
    }
    if (c.size > 1) smp_cluster_sync(); else __syncthreads();
    u64 before = (u64)(sh.scan[warp] + upto - mine);
    for (unsigned k2 = 0; k2 < c.rank; ++k2) before += smp_remote(&board->sums[0], k2);
    if (before <= n && n < before + (u64)mine) {
        u64 seen = before;
        for (int i = i0; i < i1; ++i) {
            if (__float_as_uint(e_row[i]) == tau) {
                if (seen == n) { out[r] = i; break; }
                ++seen;
            }
        }
    }
    if (c.size > 1) smp_cluster_sync();   // nobody leaves while its board may still be read
}

// How many CTAs take a row: as many as still give every CTA an SM (the kernel keeps an SM to itself), up to eight.
static int smp_cluster_for(int n_rows) {
    int sms = 148, dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int size = 1;
    while (size < SMP_MAX_CLUSTER && (long)n_rows * size * 2 <= sms) size *= 2;
    return size;
}

// scratch: float32 [n_rows, vocab] (e_i of every row).  cluster: CTAs per row (1, 2, 4 or 8), 0 lets the function choose.
IB_EXPORT int ib_sample(const float* logits, long ld, int n_rows, int vocab, const float* temperature,
                        const int* top_k, const float* top_p, const float* min_p, const float* uniform, float* scratch,
                        int cluster, int* out, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (vocab <= 0 || scratch == nullptr) return IB_ERR_ARGUMENT;
    if (cluster == 0) cluster = smp_cluster_for(n_rows);
    if (cluster != 1 && cluster != 2 && cluster != 4 && cluster != 8) return IB_ERR_ARGUMENT;
    const size_t smem = (size_t)SMP_WARPS * 256 * (sizeof(u64) + sizeof(unsigned int));
    static IbDeviceSet configured;   // the attribute is kept per device
    if (const int e = ib_allow_dynamic_smem(configured, sample_kernel, smem)) return e;
    cudaError_t e = cudaSuccess;
    for (;; cluster = 1) {   // a cluster that the device cannot place (a partitioned GPU) is tried again as single CTAs
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)n_rows * cluster);
        cfg.blockDim = dim3(SMP_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = cluster;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = ib_pdl_enabled ? 2 : 1;
        e = cudaLaunchKernelEx(&cfg, sample_kernel, logits, ld, vocab, temperature, top_k, top_p, min_p, uniform,
                               scratch, out);
        if (e == cudaSuccess || cluster == 1) break;
        (void)cudaGetLastError();
    }
    return e == cudaSuccess ? ib_launch_status() : (int)e;
}
