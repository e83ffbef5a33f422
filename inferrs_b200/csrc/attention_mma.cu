// Paged grouped-query attention on the tensor cores (bfloat16 in, float32 softmax and accumulation).
//
// One CTA works on one key/value head of one tile of query rows.  The query heads that share a
// key/value head are packed into the tile's rows: row r = (token r / G, head r % G), so the keys and
// values are read once for all G heads.  Keys are walked in tiles of 64 (whole pages), brought into
// shared memory with cp.async (zero-filled where a key is beyond the row's reach), two or three tiles in flight.
//
// Two forms of the same loop:
//   prefill form : 64 rows (64/G tokens of a prompt portion); the four warps own 16 rows each.
//   decode form  : 16 rows (one token's G heads); the four warps share the rows and take 16 keys each
//                  of every tile, and the grid's z dimension splits the keys further; partial results
//                  (unnormalised sums, row maxima, row sums) go to scratch and a second kernel merges them.
// A row at position p sees keys lo..p of its request, lo = 0 or p - window + 1.
#include "common.cuh"

#if IB_ACT_BF16

#define AM_KEYS 64
#define AM_THREADS 128
#define AM_DECODE_STAGES 3  // the decode form has little arithmetic per tile: it keeps more tiles in flight

__device__ __forceinline__ void am_cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void am_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void am_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void am_ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void am_ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3,
                                                     const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void am_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned am_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
// element offset of 16-byte chunk `chunk` of row `row` in a [rows][D] tile whose chunks are XOR-swizzled
template <int D> __device__ __forceinline__ int am_swz(int row, int chunk) {
    return row * D + ((chunk ^ (row & 7)) << 3);
}

struct AttnMmaParams {
    const __nv_bfloat16* q;        // [N, n_heads, D]
    const __nv_bfloat16* k_pages;  // [n_pages, n_kv_heads, page_size, D]
    const __nv_bfloat16* v_pages;
    const int* block_table;        // [R, max_pages]
    const int* tile_req;           // [tiles] request of the tile
    const int* tile_row0;          // [tiles] first row (token) of the tile
    const int* q_start;            // [R + 1]
    const int* positions;          // [N]
    __nv_bfloat16* out;            // [N, n_heads * D]
    float* part_o;                 // decode form with splits: [N, n_heads, splits, D]
    float* part_ml;                //                          [N, n_heads, splits, 2]
    int max_pages, page_size, n_pages, n_heads, n_kv_heads, window, n_splits;
    float scale_log2;              // scale * log2(e)
};

template <int D, bool DECODE>
__global__ void __launch_bounds__(AM_THREADS) paged_attention_mma_kernel(const AttnMmaParams P) {
    constexpr int ROWS = DECODE ? 16 : 64;
    constexpr int ST = DECODE ? AM_DECODE_STAGES : 2;  // key/value tiles in flight
    constexpr int CH = D / 8;  // 16-byte chunks per row
    extern __shared__ __align__(128) unsigned char am_smem[];
    __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(am_smem);
    __nv_bfloat16* sk = sq + ROWS * D;
    __nv_bfloat16* sv = sk + ST * AM_KEYS * D;

    ib_grid_dependency_sync();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const int tile = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int req = P.tile_req[tile], row0 = P.tile_row0[tile];
    if (req < 0) return;                            // a place in a tile list of fixed length that holds no tile
    const int G = P.n_heads / P.n_kv_heads;
    const int tpt = DECODE ? 1 : (64 / G);
    int n_tok = P.q_start[req + 1] - row0;
    if (n_tok > tpt) n_tok = tpt;
    const int p0 = P.positions[row0];
    const int pmax = p0 + n_tok - 1;
    const int lo_min = (P.window > 0 && p0 - P.window + 1 > 0) ? p0 - P.window + 1 : 0;
    const int t_first = lo_min / AM_KEYS, t_last = pmax / AM_KEYS + 1;
    int t_begin = t_first, t_end = t_last;
    if (DECODE && P.n_splits > 1) {
        const int per = (t_last - t_first + P.n_splits - 1) / P.n_splits;
        t_begin = t_first + split * per;
        t_end = t_begin + per < t_last ? t_begin + per : t_last;
    }
    const int* bt = P.block_table + (long)req * P.max_pages;

    // queries of this tile: row r = (token r / G, head r % G)
    for (int idx = tid; idx < ROWS * CH; idx += AM_THREADS) {
        const int r = idx / CH, c = idx - r * CH;
        const int ti = r / G, g = r - ti * G;
        const bool valid = ti < n_tok;
        const __nv_bfloat16* src = P.q + (((long)(row0 + (valid ? ti : 0)) * P.n_heads + kvh * G + g) * D + c * 8);
        am_cp_async16(sq + am_swz<D>(r, c), src, valid);
    }
    am_commit();

    auto load_kv = [&](int t, int buf) {
        __nv_bfloat16* dk = sk + buf * AM_KEYS * D;
        __nv_bfloat16* dv = sv + buf * AM_KEYS * D;
        for (int idx = tid; idx < AM_KEYS * CH; idx += AM_THREADS) {
            const int kk = idx / CH, c = idx - kk * CH;
            const int j = t * AM_KEYS + kk;
            bool valid = j <= pmax && j >= lo_min;
            int page = 0;
            if (valid) {
                page = bt[j / P.page_size];
                valid = page >= 0 && page < P.n_pages;
            }
            const long off = valid ? ((((long)page * P.n_kv_heads + kvh) * P.page_size + (j % P.page_size)) * D + c * 8) : 0;
            am_cp_async16(dk + am_swz<D>(kk, c), P.k_pages + off, valid);
            am_cp_async16(dv + am_swz<D>(kk, c), P.v_pages + off, valid);
        }
    };

    // per-thread rows: ra = base + gid, rb = ra + 8
    const int rbase = DECODE ? 0 : warp * 16;
    int pos_r[2], lo_r[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = rbase + gid + 8 * h;
        const int ti = r / G;
        if (ti < n_tok) {
            pos_r[h] = p0 + ti;
            lo_r[h] = (P.window > 0 && pos_r[h] - P.window + 1 > 0) ? pos_r[h] - P.window + 1 : 0;
        } else {
            pos_r[h] = -1;  // no key satisfies lo <= j <= pos
            lo_r[h] = 0;
        }
    }

    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[n][i] = 0.0f;
    float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.0f, 0.0f};

#pragma unroll
    for (int i = 0; i < ST - 1; ++i) {
        if (t_begin + i < t_end) load_kv(t_begin + i, i);
        am_commit();
    }
    am_wait<ST - 1>();  // the queries have landed
    __syncthreads();
    unsigned qf[D / 16][4];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        const int r = rbase + (lane & 7) + 8 * ((lane >> 3) & 1);
        const int c = 2 * ks + (lane >> 4);
        am_ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], sq + am_swz<D>(r, c));
    }

    constexpr int NP = DECODE ? 1 : 4;  // pairs of 8-key column tiles that this warp computes per key tile
    for (int t = t_begin; t < t_end; ++t) {
        const int buf = (t - t_begin) % ST;
        if (t + ST - 1 < t_end) load_kv(t + ST - 1, (t + ST - 1 - t_begin) % ST);  // the buffer of tile t - 1
        am_commit();
        am_wait<ST - 1>();
        __syncthreads();
        const __nv_bfloat16* tk = sk + buf * AM_KEYS * D;
        const __nv_bfloat16* tv = sv + buf * AM_KEYS * D;

        float s[2 * NP][4];
#pragma unroll
        for (int n = 0; n < 2 * NP; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[n][i] = 0.0f;
#pragma unroll
        for (int np = 0; np < NP; ++np) {
            const int key0 = DECODE ? warp * 16 : np * 16;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                unsigned b0, b1, b2, b3;
                const int kr = key0 + (lane & 7) + 8 * (lane >> 4);
                const int c = 2 * ks + ((lane >> 3) & 1);
                am_ldmatrix_x4(b0, b1, b2, b3, tk + am_swz<D>(kr, c));
                am_mma(s[2 * np], qf[ks], b0, b1);
                am_mma(s[2 * np + 1], qf[ks], b2, b3);
            }
        }
        // mask, scale, running maximum
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 2 * NP; ++n) {
            const int col0 = (DECODE ? warp * 16 : 0) + n * 8 + 2 * tig;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int h = i >> 1;
                const int j = t * AM_KEYS + col0 + (i & 1);
                const bool vis = j >= lo_r[h] && j <= pos_r[h];
                s[n][i] = vis ? s[n][i] * P.scale_log2 : -INFINITY;
                mx[h] = fmaxf(mx[h], s[n][i]);
            }
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
        for (int n = 0; n < 2 * NP; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float p = exp2f(s[n][i] - msafe[i >> 1]);  // exp2(-inf) = 0 for masked keys
                s[n][i] = p;
                l_r[i >> 1] += p;
            }
        // O += P V
#pragma unroll
        for (int kt = 0; kt < NP; ++kt) {
            unsigned a[4];
            a[0] = am_pack(s[2 * kt][0], s[2 * kt][1]);
            a[1] = am_pack(s[2 * kt][2], s[2 * kt][3]);
            a[2] = am_pack(s[2 * kt + 1][0], s[2 * kt + 1][1]);
            a[3] = am_pack(s[2 * kt + 1][2], s[2 * kt + 1][3]);
            const int key0 = DECODE ? warp * 16 : kt * 16;
#pragma unroll
            for (int dn = 0; dn < D / 16; ++dn) {
                unsigned b0, b1, b2, b3;
                const int kr = key0 + (lane & 7) + 8 * ((lane >> 3) & 1);
                const int c = 2 * dn + (lane >> 4);
                am_ldmatrix_x4_trans(b0, b1, b2, b3, tv + am_swz<D>(kr, c));
                am_mma(o[2 * dn], a, b0, b1);
                am_mma(o[2 * dn + 1], a, b2, b3);
            }
        }
        __syncthreads();  // the next iteration's loads overwrite the other buffer, which all warps have left
    }
    am_wait<0>();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_r[h] += __shfl_xor_sync(0xffffffffu, l_r[h], 1);
        l_r[h] += __shfl_xor_sync(0xffffffffu, l_r[h], 2);
    }

    if (!DECODE) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = rbase + gid + 8 * h;
            const int ti = r / G, g = r - ti * G;
            if (ti >= n_tok) continue;
            const float inv = l_r[h] > 0.0f ? 1.0f / l_r[h] : 0.0f;
            __nv_bfloat16* dst = P.out + (((long)(row0 + ti) * P.n_heads + kvh * G + g) * D);
#pragma unroll
            for (int n = 0; n < D / 8; ++n) {
                const __nv_bfloat162 v = __floats2bfloat162_rn(o[n][2 * h] * inv, o[n][2 * h + 1] * inv);
                *reinterpret_cast<__nv_bfloat162*>(dst + n * 8 + 2 * tig) = v;
            }
        }
        return;
    }

    // decode form: the four warps hold partial results over different keys of the same 16 rows
    __syncthreads();
    float* so = reinterpret_cast<float*>(sk);            // [4 warps][16 rows][D]
    float* sm = so + 4 * 16 * D;                          // [4][16]
    float* sl = sm + 4 * 16;                              // [4][16]
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = gid + 8 * h;
        if (tig == 0) { sm[warp * 16 + r] = m_r[h]; sl[warp * 16 + r] = l_r[h]; }
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            so[(warp * 16 + r) * D + n * 8 + 2 * tig] = o[n][2 * h];
            so[(warp * 16 + r) * D + n * 8 + 2 * tig + 1] = o[n][2 * h + 1];
        }
    }
    __syncthreads();
    for (int idx = tid; idx < G * D; idx += AM_THREADS) {
        const int g = idx / D, e = idx - g * D;  // row g of the tile is head g of the token
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, sm[w * 16 + g]);
        float acc = 0.0f, L = 0.0f;
        if (M > -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float f = exp2f(sm[w * 16 + g] - M);
                acc += f * so[(w * 16 + g) * D + e];
                L += f * sl[w * 16 + g];
            }
        }
        const long head = (long)row0 * P.n_heads + kvh * G + g;
        if (P.n_splits > 1) {
            P.part_o[(head * P.n_splits + split) * D + e] = acc;
            if (e == 0) {
                P.part_ml[(head * P.n_splits + split) * 2] = M;
                P.part_ml[(head * P.n_splits + split) * 2 + 1] = L;
            }
        } else {
            P.out[head * D + e] = __float2bfloat16_rn(L > 0.0f ? acc / L : 0.0f);
        }
    }
}

// out[row, head, :] = sum_s 2^(m_s - M) o_s / sum_s 2^(m_s - M) l_s
__global__ void attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                       __nv_bfloat16* __restrict__ out, int n_splits, int head_dim) {
    ib_grid_dependency_sync();
    const long head = blockIdx.x;  // row * n_heads + head
    const float* ml = part_ml + head * n_splits * 2;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, ml[2 * s]);
    for (int e = threadIdx.x; e < head_dim; e += blockDim.x) {
        float acc = 0.0f, L = 0.0f;
        if (M > -INFINITY) {
            for (int s = 0; s < n_splits; ++s) {
                const float f = exp2f(ml[2 * s] - M);
                acc += f * part_o[(head * n_splits + s) * head_dim + e];
                L += f * ml[2 * s + 1];
            }
        }
        out[head * head_dim + e] = __float2bfloat16_rn(L > 0.0f ? acc / L : 0.0f);
    }
}

template <int D, bool DECODE>
static int launch_attention_mma(const AttnMmaParams& P, int n_tiles, cudaStream_t stream) {
    constexpr int ROWS = DECODE ? 16 : 64;
    constexpr int ST = DECODE ? AM_DECODE_STAGES : 2;
    const size_t smem = (size_t)(ROWS * D + 2 * ST * AM_KEYS * D) * sizeof(__nv_bfloat16);
    static IbDeviceSet configured;   // the attribute is kept per device
    if (const int e = ib_allow_dynamic_smem(configured, paged_attention_mma_kernel<D, DECODE>, smem)) return e;
    const dim3 grid(n_tiles, P.n_kv_heads, DECODE ? P.n_splits : 1);
    ib_launch(paged_attention_mma_kernel<D, DECODE>, grid, AM_THREADS, smem, stream, P);
    return ib_launch_status();
}

// decode_form != 0: every tile is one token (n_tiles == rows of the step); n_splits >= 1 with scratch for > 1.
IB_EXPORT int ib_paged_attention_mma(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                     int max_pages, int page_size, int n_pages, const int* tile_req,
                                     const int* tile_row0, int n_tiles, const int* q_start, const int* positions,
                                     int n_rows, int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                                     void* out, int decode_form, int n_splits, float* part_o, float* part_ml,
                                     cudaStream_t stream) {
    if (n_tiles <= 0) return IB_OK;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads || page_size <= 0 || max_pages <= 0)
        return IB_ERR_ARGUMENT;
    const int G = n_heads / n_kv_heads;
    if ((head_dim != 64 && head_dim != 128 && head_dim != 256) || AM_KEYS % page_size || G > 16) return IB_ERR_UNSUPPORTED;
    if (decode_form && n_splits > 1 && (part_o == nullptr || part_ml == nullptr)) return IB_ERR_ARGUMENT;
    AttnMmaParams P;
    P.q = (const __nv_bfloat16*)q; P.k_pages = (const __nv_bfloat16*)k_pages; P.v_pages = (const __nv_bfloat16*)v_pages;
    P.block_table = block_table; P.tile_req = tile_req; P.tile_row0 = tile_row0; P.q_start = q_start;
    P.positions = positions; P.out = (__nv_bfloat16*)out; P.part_o = part_o; P.part_ml = part_ml;
    P.max_pages = max_pages; P.page_size = page_size; P.n_pages = n_pages; P.n_heads = n_heads;
    P.n_kv_heads = n_kv_heads; P.window = window; P.n_splits = decode_form ? (n_splits < 1 ? 1 : n_splits) : 1;
    P.scale_log2 = scale * 1.4426950408889634f;
    int rc;
#define IB_AM_CASE(DD)                                                                   \
    if (head_dim == DD)                                                                  \
        rc = decode_form ? launch_attention_mma<DD, true>(P, n_tiles, stream)            \
                         : launch_attention_mma<DD, false>(P, n_tiles, stream);
    IB_AM_CASE(64) else IB_AM_CASE(128) else IB_AM_CASE(256) else rc = IB_ERR_UNSUPPORTED;
#undef IB_AM_CASE
    if (rc != IB_OK) return rc;
    if (decode_form && P.n_splits > 1) {
        ib_launch(attention_merge_kernel, n_rows * n_heads, head_dim < 128 ? 64 : 128, 0, stream, (const float*)part_o,
                  (const float*)part_ml, (__nv_bfloat16*)out, P.n_splits, head_dim);
        return ib_launch_status();
    }
    return IB_OK;
}

// ---------------------------------------------------------------------------------------------
// The entry point that allocates nothing (declared and described in no_alloc.h; no counterpart in
// the reference).  Its scratch is this array in the library image; host code may not use the
// array's name as a pointer (on the host it names a stand-in, not device memory), so the device
// address is looked up once per device with cudaGetSymbolAddress and handed to the kernels.
// ---------------------------------------------------------------------------------------------
#include <mutex>

#include "no_alloc.h"

static __device__ __align__(256) float ib_noalloc_scratch[IB_NOALLOC_SCRATCH_FLOATS];

#define IB_NOALLOC_MAX_DEVICES 64
static float* g_noalloc_scratch_addr[IB_NOALLOC_MAX_DEVICES] = {nullptr};
static std::mutex g_noalloc_mutex;

// Device address of the scratch on the current device; looked up on the first call for that device.
static int noalloc_scratch(float** ptr) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= IB_NOALLOC_MAX_DEVICES) return IB_NOALLOC_ERR_ARGUMENT;
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, ib_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        g_noalloc_scratch_addr[dev] = static_cast<float*>(p);
    }
    *ptr = g_noalloc_scratch_addr[dev];
    return IB_OK;
}

IB_EXPORT int ib_paged_attention_decode_noalloc(const void* q, const void* k_pages, const void* v_pages,
                                                const int* block_table, int max_pages, int page_size, int n_pages,
                                                const int* row_request, const int* q_start, const int* positions,
                                                int n_rows, int n_heads, int n_kv_heads, int head_dim, float scale,
                                                int window, void* out, int n_splits, cudaStream_t stream) {
    if (n_rows <= 0 || n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads || head_dim <= 0 || page_size <= 0 ||
        max_pages <= 0 || n_splits <= 0)
        return IB_NOALLOC_ERR_ARGUMENT;
    const long long need = (long long)n_rows * n_heads * n_splits * (head_dim + 2);
    if (need > (long long)IB_NOALLOC_SCRATCH_FLOATS) return IB_NOALLOC_ERR_TOO_LARGE;
    float* scratch = nullptr;
    const int rc = noalloc_scratch(&scratch);
    if (rc != IB_OK) return rc;
    // the partial sums first, then the (maximum, sum) pairs, both inside the one array
    float* part_o = scratch;
    float* part_ml = scratch + (long long)n_rows * n_heads * n_splits * head_dim;
    // with one split the regular kernel writes `out` directly and touches no scratch; the scratch is
    // passed all the same so that both cases take the same path
    const int code = ib_paged_attention_mma(q, k_pages, v_pages, block_table, max_pages, page_size, n_pages,
                                            row_request, q_start, n_rows, q_start, positions, n_rows, n_heads,
                                            n_kv_heads, head_dim, scale, window, out, 1, n_splits, part_o, part_ml,
                                            stream);
    if (code == IB_ERR_UNSUPPORTED) return IB_NOALLOC_ERR_UNSUPPORTED;
    if (code == IB_ERR_ARGUMENT) return IB_NOALLOC_ERR_ARGUMENT;
    return code;
}

IB_EXPORT const char* ib_paged_attention_decode_noalloc_strerror(int code) {
    switch (code) {
        case 0: return "success";
        case IB_NOALLOC_ERR_UNSUPPORTED:
            return "sizes not taken: head_dim must be 64, 128 or 256, the page size must divide 64, and at most 16 "
                   "query heads may share a key/value head";
        case IB_NOALLOC_ERR_ARGUMENT: return "a size is zero or negative, or heads are not a multiple of kv heads";
        case IB_NOALLOC_ERR_TOO_LARGE:
            return "n_rows * n_heads * n_splits * (head_dim + 2) exceeds the built-in scratch of 4,194,304 floats";
        case IB_NOALLOC_ERR_BUILD: return "this build of the library has no bfloat16 kernels";
        default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown code";
    }
}

#else  // the float32 build has no tensor-core attention: its attention is the generic kernel

IB_EXPORT int ib_paged_attention_mma(const void*, const void*, const void*, const int*, int, int, int, const int*,
                                     const int*, int, const int*, const int*, int, int, int, int, float, int, void*,
                                     int, int, float*, float*, cudaStream_t) {
    return IB_ERR_UNSUPPORTED;
}

#include "no_alloc.h"

IB_EXPORT int ib_paged_attention_decode_noalloc(const void*, const void*, const void*, const int*, int, int, int,
                                                const int*, const int*, const int*, int, int, int, int, float, int,
                                                void*, int, cudaStream_t) {
    return IB_NOALLOC_ERR_BUILD;
}

IB_EXPORT const char* ib_paged_attention_decode_noalloc_strerror(int code) {
    return code == IB_NOALLOC_ERR_BUILD ? "this build of the library has no bfloat16 kernels" : "unknown code";
}

#endif
