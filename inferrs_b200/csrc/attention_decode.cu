// Split-KV attention for decoded tokens (one new token per request), bfloat16, head size 128.
//
// The work of one CTA is one key/value head of one request and one slice of its keys.  A producer warp
// brings the slice's keys and values page by page with TMA into a ring of 128-byte-swizzled 64-key tiles
// (no address arithmetic in the compute warps); four compute warps take 16 keys each of every tile:
// scores with mma.sync (the G query heads of the group are the rows of a 16-row tile), online softmax in
// float32, P V with mma.sync.  The warps' partial results are merged through shared memory, and the
// slices' results through float32 scratch: every CTA adds one to a counter of its (request, head group),
// and the CTA that finds it was the last one merges all slices and writes the output, so no second
// kernel is needed.  How many slices are used is decided from the request's real length (at least `min_tiles`
// tiles per slice); CTAs of unused slices leave at once.
#include <cuda.h>

#include "common.cuh"
#include "sm100.cuh"

#if IB_ACT_BF16

namespace dec {

using namespace sm100;

constexpr int D = 128;
constexpr int KEYS = 64;                    // keys per tile
constexpr int STAGES = 3;
constexpr int HALF_BYTES = KEYS * 128;      // [64 keys][64 dims] swizzled
constexpr int TILE_BYTES = 2 * HALF_BYTES;  // K or V tile
constexpr int THREADS = 160;                // 4 compute warps + producer warp

__device__ int g_error = 0;

// a bounded wait that reports through this file's error word
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, int code) {
    return mbar_wait_bounded(bar, parity, &g_error, code);
}

__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// byte offset of 16-byte chunk c (0..15 over the 128 dims) of key row `row` in a tile of two swizzled halves
__device__ __forceinline__ unsigned tile_off(int row, int c) {
    return (unsigned)((c >> 3) * HALF_BYTES + row * 128 + (((c & 7) ^ (row & 7)) << 4));
}

struct Params {
    const __nv_bfloat16* q;    // [R, n_heads, 128]
    const int* block_table;    // [R, max_pages]
    const int* positions;      // [R]
    __nv_bfloat16* out;        // [R, n_heads * 128]
    float* part_o;             // [R, n_heads, max_splits, 128]
    float* part_ml;            // [R, n_heads, max_splits, 2]
    int* counters;             // [R * n_kv_heads], zero between launches
    const int* rows;           // [R] or null: the row of q, positions and out that place i of the grid works on
    const int* reqs;           // [R] or null: its request (row of the block table); a negative row is no work
    int max_pages, page_size, n_pages, n_heads, n_kv_heads, window, max_splits, min_tiles;
    float scale_log2;
};

__global__ void __launch_bounds__(THREADS, 2) decode_kernel(const __grid_constant__ CUtensorMap map_k,
                                                            const __grid_constant__ CUtensorMap map_v, const Params P) {
    extern __shared__ unsigned char raw_smem[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~(uintptr_t)1023);
    unsigned char* sk = smem;                               // K ring
    unsigned char* sv = sk + STAGES * TILE_BYTES;           // V ring
    __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(sv + STAGES * TILE_BYTES);   // [16 rows][128], plain
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(sq + 16 * D);
    const unsigned full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    int* s_flag = reinterpret_cast<int*>(bars + 2 * STAGES);

    // Under programmatic dependent launch this kernel may start while the kernels before it still run.  What
    // they do not write is used at once: the step's description (positions, block table) and the keys and
    // values of earlier steps, so the first tiles of the ring are on their way early.  The queries and the
    // tile that holds this step's own key and value are touched only after griddepcontrol.wait.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // place i of the grid is row i of request i in a step of single tokens; in a step that also holds prompt
    // portions a list says which rows are single tokens and whose they are
    const int place = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int row = P.rows != nullptr ? P.rows[place] : place;
    // A CTA that has nothing to do still waits for the kernels before this one: a grid that has let its
    // dependents start must not complete before its own predecessors have, or the kernel after it could read
    // what they have not written yet.
    if (row < 0) { asm volatile("griddepcontrol.wait;" ::: "memory"); return; }
    const int req = P.reqs != nullptr ? P.reqs[place] : place;
    const int G = P.n_heads / P.n_kv_heads;
    const int pos = P.positions[row];
    const int lo = (P.window > 0 && pos - P.window + 1 > 0) ? pos - P.window + 1 : 0;
    const int t_first = lo / KEYS, t_last = pos / KEYS + 1;
    const int n_all = t_last - t_first;
    int n_splits = (n_all + P.min_tiles - 1) / P.min_tiles;
    if (n_splits > P.max_splits) n_splits = P.max_splits;
    if (split >= n_splits) { asm volatile("griddepcontrol.wait;" ::: "memory"); return; }   // an unused slice
    const int per = (n_all + n_splits - 1) / n_splits;
    const int t_begin = t_first + split * per;
    const int t_end = t_begin + per < t_last ? t_begin + per : t_last;
    const int n_tiles = t_end > t_begin ? t_end - t_begin : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();   // the barriers are ready: the producer starts at once
    bool ok = true;
    if (warp < 4) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        // queries of the group: rows 0..G-1, the rest of the 16 rows are zero (the four compute warps only)
        for (int idx = threadIdx.x; idx < 16 * (D / 8); idx += 128) {
            const int r = idx / (D / 8), c = idx - r * (D / 8);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < G) v = *reinterpret_cast<const uint4*>(P.q + ((long)row * P.n_heads + kvh * G + r) * D + c * 8);
            *reinterpret_cast<uint4*>(sq + r * D + c * 8) = v;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
    }

    float o[D / 8][4];
    float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.0f, 0.0f};
    const int gid = lane >> 2, tig = lane & 3;

    if (warp == 4) {
        // producer: lane p brings page p of every tile (K and V, two 64-column halves each)
        const int* bt = P.block_table + (long)req * P.max_pages;
        const int pages_per_tile = KEYS / P.page_size;
        auto lookup = [&](int i) -> int {
            if (lane >= pages_per_tile) return 0;
            const int j = (t_begin + i) * KEYS + lane * P.page_size;
            int page = (j <= pos && j / P.page_size < P.max_pages) ? bt[j / P.page_size] : -1;
            // No page (beyond the request, or given back): the copy is aimed past the last page, where TMA reads
            // nothing and fills the tile with zeros.  No query sees these keys, but their values are multiplied
            // by a probability of zero, and what an earlier owner left in a page could be no number at all.
            if (page < 0 || page >= P.n_pages) page = P.n_pages;
            return page;
        };
        int page_next = n_tiles > 0 ? lookup(0) : 0;
        // tiles that end before this step's position hold only keys of earlier steps: up to a ring of them
        // is asked for before the kernels before this one are waited for
        int n_early = pos / KEYS - t_begin;
        n_early = n_early < 0 ? 0 : (n_early > n_tiles ? n_tiles : n_early);
        n_early = n_early > STAGES ? STAGES : n_early;
        bool waited = false;
        for (int i = 0; i < n_tiles; ++i) {
            if (i == n_early) { asm volatile("griddepcontrol.wait;" ::: "memory"); waited = true; }
            const int s = i % STAGES;
            const int page = page_next;
            if (i + 1 < n_tiles) page_next = lookup(i + 1);
            if (i >= STAGES && ok && !mbar_wait(empty0 + 8 * s, ((i / STAGES) - 1) & 1, 1)) ok = false;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (lane == 0) mbar_expect_tx(full0 + 8 * s, 2 * TILE_BYTES);
            __syncwarp();
            if (lane < pages_per_tile) {
                const int grow = (page * P.n_kv_heads + kvh) * P.page_size;
                const unsigned off = (unsigned)(lane * P.page_size) * 128u;
                tma_load_2d(smem_u32(sk + s * TILE_BYTES) + off, &map_k, 0, grow, full0 + 8 * s);
                tma_load_2d(smem_u32(sk + s * TILE_BYTES + HALF_BYTES) + off, &map_k, 64, grow, full0 + 8 * s);
                tma_load_2d(smem_u32(sv + s * TILE_BYTES) + off, &map_v, 0, grow, full0 + 8 * s);
                tma_load_2d(smem_u32(sv + s * TILE_BYTES + HALF_BYTES) + off, &map_v, 64, grow, full0 + 8 * s);
            }
        }
        if (!waited) asm volatile("griddepcontrol.wait;" ::: "memory");   // the loop never reached it
    } else {
#pragma unroll
        for (int n = 0; n < D / 8; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) o[n][i] = 0.0f;
        // query fragments: rows gid and gid + 8 of the 16-row tile
        unsigned qf[D / 16][4];
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            const int r = (lane & 7) + 8 * ((lane >> 3) & 1);
            const int c = 2 * ks + (lane >> 4);
            ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], smem_u32(sq + r * D + c * 8));
        }
        const bool row_ok[2] = {gid < G, gid + 8 < G};
        for (int i = 0; i < n_tiles; ++i) {
            const int s = i % STAGES;
            if (ok && !mbar_wait(full0 + 8 * s, (i / STAGES) & 1, 2)) ok = false;
            const unsigned tk = smem_u32(sk + s * TILE_BYTES), tv = smem_u32(sv + s * TILE_BYTES);
            const int key0 = warp * 16;                      // this warp's 16 keys of the tile
            float sc[2][4];
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) sc[n][e] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                unsigned b0, b1, b2, b3;
                const int kr = key0 + (lane & 7) + 8 * (lane >> 4);
                const int c = 2 * ks + ((lane >> 3) & 1);
                ldmatrix_x4(b0, b1, b2, b3, tk + tile_off(kr, c));
                mma16816(sc[0], qf[ks], b0, b1);
                mma16816(sc[1], qf[ks], b2, b3);
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int h = e >> 1;
                    const int j = (t_begin + i) * KEYS + key0 + n * 8 + 2 * tig + (e & 1);
                    const bool vis = row_ok[h] && j >= lo && j <= pos;
                    sc[n][e] = vis ? sc[n][e] * P.scale_log2 : -INFINITY;
                    mx[h] = fmaxf(mx[h], sc[n][e]);
                }
            float corr[2], msafe[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                const float m_new = fmaxf(m_r[h], mx[h]);
                msafe[h] = m_new == -INFINITY ? 0.0f : m_new;
                corr[h] = m_r[h] == -INFINITY ? 0.0f : exp2f(m_r[h] - msafe[h]);
                m_r[h] = m_new;
                l_r[h] *= corr[h];
            }
#pragma unroll
            for (int n = 0; n < D / 8; ++n) {
                o[n][0] *= corr[0]; o[n][1] *= corr[0];
                o[n][2] *= corr[1]; o[n][3] *= corr[1];
            }
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p = exp2f(sc[n][e] - msafe[e >> 1]);
                    sc[n][e] = p;
                    l_r[e >> 1] += p;
                }
            unsigned a[4];
            a[0] = pack_bf16(sc[0][0], sc[0][1]);
            a[1] = pack_bf16(sc[0][2], sc[0][3]);
            a[2] = pack_bf16(sc[1][0], sc[1][1]);
            a[3] = pack_bf16(sc[1][2], sc[1][3]);
#pragma unroll
            for (int dn = 0; dn < D / 16; ++dn) {
                unsigned b0, b1, b2, b3;
                const int kr = key0 + (lane & 7) + 8 * ((lane >> 3) & 1);
                const int c = 2 * dn + (lane >> 4);
                ldmatrix_x4_trans(b0, b1, b2, b3, tv + tile_off(kr, c));
                mma16816(o[2 * dn], a, b0, b1);
                mma16816(o[2 * dn + 1], a, b2, b3);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * s);      // this warp has read the stage
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            l_r[h] += __shfl_xor_sync(0xffffffffu, l_r[h], 1);
            l_r[h] += __shfl_xor_sync(0xffffffffu, l_r[h], 2);
        }
    }

    // merge the four warps' partial results (different keys, same rows); the rings are idle by now
    __syncthreads();
    float* so = reinterpret_cast<float*>(sk);                // [4 warps][16 rows][128]
    float* sm = so + 4 * 16 * D;                              // [4][16]
    float* sl = sm + 4 * 16;                                  // [4][16]
    if (warp < 4) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = gid + 8 * h;
            if (r >= G) continue;                             // rows beyond the group's heads hold nothing
            if (tig == 0) { sm[warp * 16 + r] = m_r[h]; sl[warp * 16 + r] = l_r[h]; }
#pragma unroll
            for (int n = 0; n < D / 8; ++n) {
                *reinterpret_cast<float2*>(so + (warp * 16 + r) * D + n * 8 + 2 * tig) = make_float2(o[n][2 * h], o[n][2 * h + 1]);
            }
        }
    }
    __syncthreads();
    const long head0 = (long)row * P.n_heads + kvh * G;       // of q and out
    const long part0 = (long)place * P.n_heads + kvh * G;     // of the slices' scratch
    for (int idx = threadIdx.x; idx < G * (D / 4); idx += THREADS) {   // four elements per thread: one pass
        const int g = idx / (D / 4), e = (idx - g * (D / 4)) * 4;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, sm[w * 16 + g]);
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        float L = 0.0f;
        if (M > -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float f = exp2f(sm[w * 16 + g] - M);
                const float4 v = *reinterpret_cast<const float4*>(so + (w * 16 + g) * D + e);
                acc.x += f * v.x; acc.y += f * v.y; acc.z += f * v.z; acc.w += f * v.w;
                L += f * sl[w * 16 + g];
            }
        }
        if (n_splits > 1) {
            *reinterpret_cast<float4*>(P.part_o + ((part0 + g) * P.max_splits + split) * D + e) = acc;
            if (e == 0) {
                P.part_ml[((part0 + g) * P.max_splits + split) * 2] = M;
                P.part_ml[((part0 + g) * P.max_splits + split) * 2 + 1] = L;
            }
        } else {
            if (!(L > 0.0f)) { acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f); L = 1.0f; }
            __nv_bfloat162 lo2 = __floats2bfloat162_rn(acc.x / L, acc.y / L);
            __nv_bfloat162 hi2 = __floats2bfloat162_rn(acc.z / L, acc.w / L);
            uint2 w2;
            w2.x = *reinterpret_cast<unsigned*>(&lo2);
            w2.y = *reinterpret_cast<unsigned*>(&hi2);
            *reinterpret_cast<uint2*>(P.out + (head0 + g) * D + e) = w2;
        }
    }
    if (n_splits > 1) {
        // the slice that arrives last merges them all
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            const int old = atomicAdd(P.counters + place * P.n_kv_heads + kvh, 1);
            *s_flag = old == n_splits - 1;
            if (old == n_splits - 1) P.counters[place * P.n_kv_heads + kvh] = 0;   // zero again for the next launch
        }
        __syncthreads();
        if (*s_flag) {
            __threadfence();
            // four output elements per thread, all slices' parts asked for before the first is used
            for (int idx = threadIdx.x; idx < G * (D / 4); idx += THREADS) {
                const int g = idx / (D / 4), e = (idx - g * (D / 4)) * 4;
                const float* ml = P.part_ml + (part0 + g) * P.max_splits * 2;
                const float* po = P.part_o + (part0 + g) * P.max_splits * D + e;
                constexpr int MAX_SLICES = 8;   // more slices go through the loop below in groups of eight
                float M = -INFINITY;
                for (int s = 0; s < n_splits; ++s) M = fmaxf(M, __ldcg(ml + 2 * s));
                float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                float L = 0.0f;
                if (M > -INFINITY) {
                    for (int s0 = 0; s0 < n_splits; s0 += MAX_SLICES) {
                        float4 part[MAX_SLICES];
                        float mm[MAX_SLICES], ll[MAX_SLICES];
#pragma unroll
                        for (int j = 0; j < MAX_SLICES; ++j) {
                            const bool live = s0 + j < n_splits;
                            part[j] = live ? __ldcg(reinterpret_cast<const float4*>(po + (long)(s0 + j) * D))
                                           : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                            mm[j] = live ? __ldcg(ml + 2 * (s0 + j)) : -INFINITY;
                            ll[j] = live ? __ldcg(ml + 2 * (s0 + j) + 1) : 0.0f;
                        }
#pragma unroll
                        for (int j = 0; j < MAX_SLICES; ++j) {
                            const float f = exp2f(mm[j] - M);
                            acc.x += f * part[j].x; acc.y += f * part[j].y; acc.z += f * part[j].z; acc.w += f * part[j].w;
                            L += f * ll[j];
                        }
                    }
                }
                if (!(L > 0.0f)) { acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f); L = 1.0f; }
                __nv_bfloat162 lo2 = __floats2bfloat162_rn(acc.x / L, acc.y / L);
                __nv_bfloat162 hi2 = __floats2bfloat162_rn(acc.z / L, acc.w / L);
                uint2 w;
                w.x = *reinterpret_cast<unsigned*>(&lo2);
                w.y = *reinterpret_cast<unsigned*>(&hi2);
                *reinterpret_cast<uint2*>(P.out + (head0 + g) * D + e) = w;
            }
        }
    }
    if (!ok) {   // a wait of this CTA ran out: let its copies land before the shared memory is given back
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
}

}  // namespace dec

// One new token per request: row r = request r, or, with `rows` and `reqs` (n_rows entries each), row rows[i] of
// request reqs[i] (a negative row is skipped).  part_o [rows, n_heads, max_splits, 128] and part_ml
// [rows, n_heads, max_splits, 2] are float32 scratch; counters [rows * n_kv_heads] are ints that are zero
// (the kernel leaves them zero).  Launches that share scratch and counters must not overlap.
IB_EXPORT int ib_paged_attention_decode(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                        int max_pages, int page_size, int n_pages, const int* positions, int n_rows,
                                        int n_heads, int n_kv_heads, int head_dim, float scale, int window, void* out,
                                        int max_splits, int min_tiles, float* part_o, float* part_ml, int* counters,
                                        const int* rows, const int* reqs, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (min_tiles <= 0) return IB_ERR_ARGUMENT;
    if ((rows == nullptr) != (reqs == nullptr)) return IB_ERR_ARGUMENT;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads || page_size <= 0 || max_pages <= 0 || max_splits <= 0)
        return IB_ERR_ARGUMENT;
    const int G = n_heads / n_kv_heads;
    if (head_dim != dec::D || dec::KEYS % page_size || page_size < 8 || G > 16) return IB_ERR_UNSUPPORTED;
    if (max_splits > 1 && (part_o == nullptr || part_ml == nullptr || counters == nullptr)) return IB_ERR_ARGUMENT;
    dec::EncodeTiled enc = dec::encode_fn();
    if (enc == nullptr) return IB_ERR_UNSUPPORTED;
    CUtensorMap mk, mv;
    for (int which = 0; which < 2; ++which) {
        const cuuint64_t dims[2] = {128, (cuuint64_t)n_pages * n_kv_heads * page_size};
        const cuuint64_t strides[1] = {128 * 2};
        const cuuint32_t box[2] = {64, (cuuint32_t)page_size};
        const cuuint32_t elem[2] = {1, 1};
        if (enc(which ? &mv : &mk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(which ? v_pages : k_pages), dims,
                strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return IB_ERR_UNSUPPORTED;
    }
    dec::Params P;
    P.q = (const __nv_bfloat16*)q; P.block_table = block_table; P.positions = positions; P.out = (__nv_bfloat16*)out;
    P.part_o = part_o; P.part_ml = part_ml; P.counters = counters; P.rows = rows; P.reqs = reqs;
    P.max_pages = max_pages; P.page_size = page_size;
    P.n_pages = n_pages; P.n_heads = n_heads; P.n_kv_heads = n_kv_heads; P.window = window; P.max_splits = max_splits;
    P.min_tiles = min_tiles;
    P.scale_log2 = scale * 1.4426950408889634f;
    const size_t smem = 2 * dec::STAGES * dec::TILE_BYTES + 16 * dec::D * 2 + (2 * dec::STAGES + 1) * 8 + 1024;
    static IbDeviceSet configured;   // the attribute is kept per device
    if (const int e = ib_allow_dynamic_smem(configured, dec::decode_kernel, smem)) return e;
    ib_launch(dec::decode_kernel, dim3(n_rows, n_kv_heads, max_splits), dec::THREADS, smem, stream, mk, mv, P);
    return ib_launch_status();
}

IB_EXPORT int ib_attention_decode_error(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, dec::g_error, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(dec::g_error, &zero, sizeof(int));
    }
    return v;
}

// The same word on its way to `out` (pinned host memory) in stream order, without waiting for the device: the
// caller reads it after an event that it records behind this call.
IB_EXPORT int ib_attention_decode_error_async(int* out, cudaStream_t stream) {
    return (int)cudaMemcpyFromSymbolAsync(out, dec::g_error, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
}

#else

IB_EXPORT int ib_paged_attention_decode(const void*, const void*, const void*, const int*, int, int, int, const int*, int,
                                        int, int, int, float, int, void*, int, int, float*, float*, int*, const int*,
                                        const int*, cudaStream_t) {
    return IB_ERR_UNSUPPORTED;
}

IB_EXPORT int ib_attention_decode_error(int) { return 0; }

IB_EXPORT int ib_attention_decode_error_async(int* out, cudaStream_t) { *out = 0; return 0; }

#endif
