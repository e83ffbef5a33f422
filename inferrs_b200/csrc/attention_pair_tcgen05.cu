// Paged grouped-query attention for prompt portions on tcgen05 tensor cores (bfloat16, head size 128): two query
// tiles per CTA that take turns, probabilities handed to the second product through tensor memory.
//
// One CTA owns 256 query rows of one key/value head as two tiles of 128 rows: tile t holds 128/G consecutive
// tokens of one request with the G query heads that share the key/value head side by side (row = token * G +
// head); tile 1 continues where tile 0 ends.  Keys are walked in tiles of 128 (whole pages), and every key and
// value tile that arrives serves both query tiles.  Per key tile and query tile:
//   S  = Q K^T   128 lanes x 128 columns of float32 in tensor memory, one such region per query tile;
//   P  = exp2(S * scale - m) by ONE thread per row: it reads its row of S with tcgen05.ld in pieces of 32
//        columns (once for the row's maximum, once for the exponentials), keeps the reference maximum m and the
//        sum in float32 and writes P as bfloat16 pairs with tcgen05.st over the first 64 columns of the same
//        region: the probabilities never pass through shared memory;
//   O += P V     with P read from tensor memory as the A operand and V from shared memory as MN-major B,
//        accumulated in tensor memory over all key tiles (128 lanes x 128 columns per query tile) and read once at
//        the end.  The reference maximum of a row moves only when the row's maximum has grown by more than 8 (a
//        factor of 256) since it was set; then the row of O and the sum are scaled to the new reference first.
//        Until then P may reach 256, which bfloat16 and the float32 sums hold as well as values below 1, so the
//        result is the same softmax.
// Shared memory carries only what the tensor cores read from it (Q twice 32 KB, K and V two stages of 32 KB each):
// with both operands of both products and the probabilities in shared memory its bandwidth, not the tensor
// pipe, bounds a kernel of this shape.  One thread issues all products, in an order that lets the two query
// tiles take turns: while one tile's threads compute exponentials, the tensor pipe multiplies for the other.
//   Q K0(0), Q K1(0); then per key tile i: [P V0(i), Q K0(i + 1)], [P V1(i), Q K1(i + 1)]
// Products run in the order of issue, so Q Kt(i + 1) may overwrite the region that P Vt(i) reads P from.
//
// Warps 0..3: softmax and output of query tile 0 (warp w: lanes 32 w ..); warps 4..7: of query tile 1; warp 8:
// TMA producer of Q and K; warp 9: issuer of all products and owner of the tensor-memory allocation; warp 10: TMA
// producer of V; warp 11: idle.  All mbarrier waits are bounded (about two seconds) and report through the library's
// error word.
#include <cuda.h>

#include "common.cuh"
#include "sm100.cuh"

#if IB_ACT_BF16

namespace fp {

using namespace sm100;

constexpr int D = 128;                 // head size
constexpr int ROWS = 128;              // rows of a query tile
constexpr int KEYS = 128;              // keys per tile
constexpr int THREADS = 384;
constexpr int SMEM_SLACK = 1024;       // bytes that the 1 KB alignment of the tiles may cost
constexpr int HALF_BYTES = 128 * 128;  // [128 rows][64 elements] swizzled sub-tile
constexpr int TILE_BYTES = 2 * HALF_BYTES;   // a Q, K or V tile: 128 x 128 bfloat16
constexpr float RESCALE_STEP = 8.0f;   // how far a row's maximum may outgrow its reference (in powers of two)

__device__ int g_error = 0;

// a bounded wait that reports through this file's error word
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, int code) {
    return mbar_wait_bounded(bar, parity, &g_error, code);
}

// three-input maximum, and two float32 operations in one instruction (sm_100)
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ float2 fma2(float x0, float x1, float scale, float add) {   // (x0, x1) * scale + add
    unsigned long long x, sc, ad, d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(x) : "f"(x0), "f"(x1));
    asm("mov.b64 %0, {%1, %1};" : "=l"(sc) : "f"(scale));
    asm("mov.b64 %0, {%1, %1};" : "=l"(ad) : "f"(add));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(x), "l"(sc), "l"(ad));
    float2 r;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(d));
    return r;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    unsigned long long x, y, d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(x) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(y) : "f"(b.x), "f"(b.y));
    asm("add.f32x2 %0, %1, %2;" : "=l"(d) : "l"(x), "l"(y));
    float2 r;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(d));
    return r;
}

struct Params {
    const int* block_table;   // [R, max_pages]
    const int* tile_req;      // [tiles]
    const int* tile_row0;     // [tiles] first token row of the tile
    const int* q_start;       // [R + 1]
    const int* positions;     // [N]
    __nv_bfloat16* out;       // [N, n_heads * 128]
    int max_pages, page_size, n_pages, n_heads, n_kv_heads, window;
    float scale_log2;
};

__global__ void __launch_bounds__(THREADS, 1) attention_pair_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                    const __grid_constant__ CUtensorMap map_k,
                                                                    const __grid_constant__ CUtensorMap map_v,
                                                                    const Params P) {
    extern __shared__ __align__(1024) unsigned char raw_smem[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~(uintptr_t)1023);
    unsigned char* sq = smem;                       // Q tiles 0 and 1
    unsigned char* sk = sq + 2 * TILE_BYTES;        // K tiles, two stages
    unsigned char* sv = sk + 2 * TILE_BYTES;        // V tiles, two stages
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(sv + 2 * TILE_BYTES);
    const unsigned q_full = smem_u32(bars);
    const unsigned k_full0 = smem_u32(bars + 1), k_empty0 = smem_u32(bars + 3);
    const unsigned v_full0 = smem_u32(bars + 5), v_empty0 = smem_u32(bars + 7);
    const unsigned s_full0 = smem_u32(bars + 9);    // per query tile: S of the next key tile is there
    const unsigned p_full0 = smem_u32(bars + 11);   // per query tile and half of the key tile (2 t + h): its P is there
    const unsigned h_done0 = smem_u32(bars + 15);   // per query tile: the products of the key tile's first half are done
    const unsigned o_full0 = smem_u32(bars + 17);   // per query tile: O holds every key tile
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 19);

    ib_grid_dependency_sync();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // The last tiles of a prompt see the most keys: they are started first, so that the grid's tail is short.  Blocks
    // are handed out in the order of their index, so the index counts tiles from the last one down and the
    // key/value heads within each tile (with the heads as a second grid dimension all tiles of head 0, short ones
    // included, would come before the long tiles of the other heads).
    const int tile = (int)(gridDim.x / P.n_kv_heads) - 1 - (int)(blockIdx.x / P.n_kv_heads);
    const int kvh = (int)(blockIdx.x % P.n_kv_heads);
    const int req = P.tile_req[tile], row0 = P.tile_row0[tile];
    if (req < 0) return;                            // a place in a tile list of fixed length that holds no tile
    const int G = P.n_heads / P.n_kv_heads;
    const int tpt = ROWS / G;                       // tokens per query tile (a group size that does not divide 128 leaves rows unused)
    int n_tok = P.q_start[req + 1] - row0;          // tokens of both query tiles
    if (n_tok > 2 * tpt) n_tok = 2 * tpt;
    const int p0 = P.positions[row0];
    // key tiles that each query tile walks: from the first one that its first token's window reaches (the same
    // for both: the earlier tile's) to the one that holds its last token
    const int lo_min = (P.window > 0 && p0 - P.window + 1 > 0) ? p0 - P.window + 1 : 0;
    const int t_begin = lo_min / KEYS;
    const int n_tok_t[2] = {n_tok < tpt ? n_tok : tpt, n_tok > tpt ? n_tok - tpt : 0};
    int n_tiles_t[2];
    n_tiles_t[0] = (p0 + n_tok_t[0] - 1) / KEYS + 1 - t_begin;
    n_tiles_t[1] = n_tok_t[1] > 0 ? (p0 + n_tok - 1) / KEYS + 1 - t_begin : 0;
    const int n_tiles = n_tiles_t[0] > n_tiles_t[1] ? n_tiles_t[0] : n_tiles_t[1];
    const int pmax = p0 + n_tok - 1;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(k_full0 + 8 * s, 1); mbar_init(k_empty0 + 8 * s, 1);
            mbar_init(v_full0 + 8 * s, 1); mbar_init(v_empty0 + 8 * s, 1);
            mbar_init(s_full0 + 8 * s, 1); mbar_init(o_full0 + 8 * s, 1); mbar_init(h_done0 + 8 * s, 1);
            mbar_init(p_full0 + 16 * s, 4); mbar_init(p_full0 + 16 * s + 8, 4);   // four warps arrive
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before();
    __syncthreads();
    fence_after();
    const unsigned tmem = *tmem_slot;      // columns 128 t: S and P of query tile t; 256 + 128 t: O of tile t
    bool ok = true;

    if (warp == 8 || warp == 10) {
        // TMA producers: warp 8 brings the queries and the key tiles, warp 10 the value tiles.  Lane p brings page
        // p of every tile (two boxes: the 64-column halves) and looks the page up one tile ahead of its use.
        if (warp == 8 && lane == 0) {
            const int n_q = n_tok_t[1] > 0 ? 2 : 1;
            mbar_expect_tx(q_full, n_q * tpt * G * 256);   // per tile [tokens][G heads][128] as two 64-column halves
            for (int t = 0; t < n_q; ++t) {
                tma_load_3d(smem_u32(sq + t * TILE_BYTES), &map_q, 0, kvh * G, row0 + t * tpt, q_full);
                tma_load_3d(smem_u32(sq + t * TILE_BYTES + HALF_BYTES), &map_q, 64, kvh * G, row0 + t * tpt, q_full);
            }
        }
        const int* bt = P.block_table + (long)req * P.max_pages;
        const int pages_per_tile = KEYS / P.page_size;   // at most 16
        auto lookup = [&](int i) -> int {
            if (lane >= pages_per_tile) return 0;
            const int j = (t_begin + i) * KEYS + lane * P.page_size;
            int page = (j <= pmax && j / P.page_size < P.max_pages) ? bt[j / P.page_size] : -1;
            // No page (beyond the request, or given back): the copy is aimed past the last page, where TMA reads
            // nothing and fills the tile with zeros.  No query sees these keys, but their values are multiplied
            // by a probability of zero, and what an earlier owner left in a page could be no number at all.
            if (page < 0 || page >= P.n_pages) page = P.n_pages;
            return page;
        };
        const bool keys = warp == 8;
        const unsigned full0 = keys ? k_full0 : v_full0, empty0 = keys ? k_empty0 : v_empty0;
        int page = n_tiles > 0 ? lookup(0) : 0;
        for (int i = 0; i < n_tiles; ++i) {
            const int page_next = i + 1 < n_tiles ? lookup(i + 1) : 0;
            const int s = i & 1;
            if (i >= 2 && ok && !mbar_wait(empty0 + 8 * s, ((i >> 1) - 1) & 1, 1)) ok = false;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (lane == 0) mbar_expect_tx(full0 + 8 * s, TILE_BYTES);
            __syncwarp();
            if (lane < pages_per_tile) {
                const int grow = (page * P.n_kv_heads + kvh) * P.page_size;
                const unsigned off = (unsigned)(lane * P.page_size) * 128u;
                unsigned char* dst = (keys ? sk : sv) + s * TILE_BYTES;
                tma_load_2d(smem_u32(dst) + off, keys ? &map_k : &map_v, 0, grow, full0 + 8 * s);
                tma_load_2d(smem_u32(dst + HALF_BYTES) + off, keys ? &map_k : &map_v, 64, grow, full0 + 8 * s);
            }
            page = page_next;
        }
    } else if (warp == 9) {
        // Both products: M = 128, N = 128, bfloat16 in, float32 out.  S = Q K^T takes both operands from shared memory
        // (K-major); O += P V takes P from tensor memory and V from shared memory as MN-major B.
        const unsigned idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(KEYS >> 3) << 17) | ((unsigned)(ROWS >> 4) << 24);
        const unsigned idesc_pv = idesc_qk | (1u << 16);
        if (lane == 0 && n_tiles > 0) {
            auto issue_qk = [&](int t, int i) {       // S_t = Q_t K(i)^T
                const int s = i & 1;
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const unsigned off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
                    umma(tmem + t * 128, desc_k_major(smem_u32(sq + t * TILE_BYTES) + off),
                         desc_k_major(smem_u32(sk + s * TILE_BYTES) + off), idesc_qk, k != 0);
                }
                umma_commit(s_full0 + 8 * t);
            };
            // O_t += P_t V(i) over one half of the key tile: 16 keys are 8 columns of P and 16 rows of V
            auto issue_pv = [&](int t, int i, int h) {
                const int s = i & 1;
#pragma unroll
                for (int k = 4 * h; k < 4 * h + 4; ++k)
                    umma_ts(tmem + 256 + t * 128, tmem + t * 128 + k * 8,
                            desc_mn_major(smem_u32(sv + s * TILE_BYTES) + k * 16 * 128, HALF_BYTES), idesc_pv, (i | k) != 0);
            };
            if (!mbar_wait(q_full, 0, 2)) ok = false;
            if (ok && !mbar_wait(k_full0, 0, 2)) ok = false;
            if (ok) {
                fence_after();
                for (int t = 0; t < 2; ++t)
                    if (n_tiles_t[t] > 0) issue_qk(t, 0);
                umma_commit(k_empty0);                  // K(0) is free once these products are done
            }
            for (int i = 0; i < n_tiles && ok; ++i) {
                const int s = i & 1;
                bool have_v = false, have_k = false;
                for (int t = 0; t < 2 && ok; ++t) {
                    if (i < n_tiles_t[t]) {
                        // the first half's products run while the row's threads still compute the second half's P
                        if (!mbar_wait(p_full0 + 16 * t, i & 1, 4)) { ok = false; break; }
                        if (!have_v && !mbar_wait(v_full0 + 8 * s, (i >> 1) & 1, 3)) { ok = false; break; }
                        have_v = true;
                        fence_after();
                        issue_pv(t, i, 0);
                        umma_commit(h_done0 + 8 * t);
                        if (!mbar_wait(p_full0 + 16 * t + 8, i & 1, 4)) { ok = false; break; }
                        fence_after();
                        issue_pv(t, i, 1);
                        if (i == n_tiles_t[t] - 1) umma_commit(o_full0 + 8 * t);
                    }
                    if (i + 1 < n_tiles_t[t]) {
                        if (!have_k && !mbar_wait(k_full0 + 8 * (s ^ 1), ((i + 1) >> 1) & 1, 2)) { ok = false; break; }
                        have_k = true;
                        fence_after();
                        issue_qk(t, i + 1);
                    }
                }
                if (!ok) break;
                umma_commit(v_empty0 + 8 * s);                      // V(i) is free once these products are done
                if (i + 1 < n_tiles) umma_commit(k_empty0 + 8 * (s ^ 1));   // and K(i + 1)
            }
        }
    } else if (warp < 8) {
        // softmax and output: one thread per row of its query tile
        const int t = warp >> 2;
        const int r = (warp & 3) * 32 + lane;
        const int ti = r / G, g = r - ti * G;
        const bool row_valid = ti < n_tok_t[t];
        const int pos = row_valid ? p0 + t * tpt + ti : -1;
        const int lo = (row_valid && P.window > 0 && pos - P.window + 1 > 0) ? pos - P.window + 1 : 0;
        const unsigned lane_addr = (unsigned)((warp & 3) * 32) << 16;
        const unsigned s_addr = tmem + lane_addr + t * 128;
        const unsigned o_addr = tmem + lane_addr + 256 + t * 128;
        float m_ref = -INFINITY, l = 0.0f;   // the reference that P and O are scaled to, and the sum of P
        const int my_tiles = n_tiles_t[t];
        for (int i = 0; i < my_tiles; ++i) {
            if (ok && !mbar_wait(s_full0 + 8 * t, i & 1, 5)) ok = false;
            ok = __all_sync(0xffffffffu, ok);   // the tensor-memory loads and stores below are warp-wide
            if (!ok) break;
            fence_after();
            const int key0 = (t_begin + i) * KEYS;
            // The key tile goes in two halves of 64 keys: the second product starts on the first half's P while the
            // second half's exponentials are computed.
#pragma unroll 1
            for (int h = 0; h < 2 && ok; ++h) {
                const int kbase = key0 + 64 * h;
                unsigned a[32], b[32];
                tmem_ld32_issue(s_addr + 64 * h, a);
                tmem_ld32_issue(s_addr + 64 * h + 32, b);
                tmem_ld_wait();
                // a half whose keys this row sees in full needs no comparisons (all but the first and last few)
                const bool all_visible = kbase >= lo && kbase + 63 <= pos;
                if (!all_visible) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int ka = kbase + j, kb = ka + 32;
                        if (!(ka >= lo && ka <= pos)) a[j] = 0xff800000u;   // -inf: exp2 gives 0
                        if (!(kb >= lo && kb <= pos)) b[j] = 0xff800000u;
                    }
                }
                // the row's maximum over the half (four chains of three-input maxima)
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    mx4[j & 3] = max3(mx4[j & 3], __uint_as_float(a[2 * j]), __uint_as_float(a[2 * j + 1]));
                    mx4[(j + 2) & 3] = max3(mx4[(j + 2) & 3], __uint_as_float(b[2 * j]), __uint_as_float(b[2 * j + 1]));
                }
                const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * P.scale_log2;   // the scale is positive
                // Move the reference?  Only if the maximum has outgrown it by more than the step (or there is none yet).
                const bool move = mx > m_ref + RESCALE_STEP || (m_ref == -INFINITY && mx > -INFINITY);
                if ((i | h) != 0 && __any_sync(0xffffffffu, move)) {
                    // O must stand still while its rows are scaled.  First half: S of this tile is there, so every
                    // product issued before it is done and none is issued until this half's P is handed over.  Second
                    // half: the first half's products, which were started a moment ago, have to be done.
                    if (h == 1 && !mbar_wait(h_done0 + 8 * t, i & 1, 6)) ok = false;
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    fence_after();
                    const float corr = move ? (m_ref == -INFINITY ? 0.0f : ex2(m_ref - mx)) : 1.0f;
#pragma unroll 1
                    for (int c = 0; c < D; c += 32) {
                        unsigned v[32];
                        tmem_ld32_issue(o_addr + c, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * corr);
                        tmem_st32(o_addr + c, v);
                    }
                    l *= corr;
                }
                if (move) m_ref = mx;
                const float neg_m = m_ref == -INFINITY ? 0.0f : -m_ref;
                // P = exp2(S * scale - m) as bfloat16 pairs, written over columns of S that have been read
                float2 sum2[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
                unsigned w[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    float2 x = fma2(__uint_as_float(a[2 * j]), __uint_as_float(a[2 * j + 1]), P.scale_log2, neg_m);
                    x.x = ex2(x.x); x.y = ex2(x.y);
                    sum2[j & 1] = add2(sum2[j & 1], x);
                    w[j] = pack_bf16(x.x, x.y);
                }
                tmem_st16(s_addr + 32 * h, w);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    float2 x = fma2(__uint_as_float(b[2 * j]), __uint_as_float(b[2 * j + 1]), P.scale_log2, neg_m);
                    x.x = ex2(x.x); x.y = ex2(x.y);
                    sum2[j & 1] = add2(sum2[j & 1], x);
                    w[j] = pack_bf16(x.x, x.y);
                }
                tmem_st16(s_addr + 32 * h + 16, w);
                l += (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
                // this half's P is written (and O scaled, if it was): tell the issuer (one arrival per warp)
                tmem_st_wait();
                fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full0 + 16 * t + 8 * h);
            }
            if (!ok) break;
        }
        if (ok && my_tiles > 0) {
            if (!mbar_wait(o_full0 + 8 * t, 0, 6)) ok = false;
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
                fence_after();
                const float inv = l > 0.0f ? 1.0f / l : 0.0f;
                __nv_bfloat16* dst = P.out + ((long)(row0 + t * tpt + ti) * P.n_heads + kvh * G + g) * D;
#pragma unroll 1
                for (int c = 0; c < D; c += 32) {
                    unsigned v[32];
                    tmem_ld32_issue(o_addr + c, v);
                    tmem_ld_wait();
                    if (row_valid) {
#pragma unroll
                        for (int c0 = 0; c0 < 32; c0 += 8) {
                            uint4 w;
                            w.x = pack_bf16(__uint_as_float(v[c0]) * inv, __uint_as_float(v[c0 + 1]) * inv);
                            w.y = pack_bf16(__uint_as_float(v[c0 + 2]) * inv, __uint_as_float(v[c0 + 3]) * inv);
                            w.z = pack_bf16(__uint_as_float(v[c0 + 4]) * inv, __uint_as_float(v[c0 + 5]) * inv);
                            w.w = pack_bf16(__uint_as_float(v[c0 + 6]) * inv, __uint_as_float(v[c0 + 7]) * inv);
                            *reinterpret_cast<uint4*>(dst + c + c0) = w;
                        }
                    }
                }
            }
        }
    }

    if (!ok) {   // a wait of this CTA ran out: copies still in flight get time to land before it leaves
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    fence_before();
    __syncthreads();
    if (warp == 9) {
        fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

}  // namespace fp

// Prefill-form attention for head size 128, bfloat16: tile i holds up to 2 * 128/G tokens of request tile_req[i]
// from row tile_row0[i].  Same arguments and results as ib_paged_attention_tcgen05, whose tiles hold half as many.
IB_EXPORT int ib_paged_attention_pair_tcgen05(const void* q, const void* k_pages, const void* v_pages,
                                              const int* block_table, int max_pages, int page_size, int n_pages,
                                              const int* tile_req, const int* tile_row0, int n_tiles, const int* q_start,
                                              const int* positions, int n_rows, int n_heads, int n_kv_heads, int head_dim,
                                              float scale, int window, void* out, cudaStream_t stream) {
    if (n_tiles <= 0) return IB_OK;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads || page_size <= 0 || max_pages <= 0) return IB_ERR_ARGUMENT;
    const int G = n_heads / n_kv_heads;
    if (head_dim != fp::D || fp::KEYS % page_size || page_size < 8 || G > fp::ROWS) return IB_ERR_UNSUPPORTED;
    if (!(scale > 0.0f)) return IB_ERR_UNSUPPORTED;   // the row maximum is taken before the scale is applied
    sm100::EncodeTiled enc = sm100::encode_fn();
    if (enc == nullptr) return IB_ERR_UNSUPPORTED;
    CUtensorMap mq, mk, mv;
    {
        // q [n_rows tokens][n_heads][128]: boxes of [128/G tokens][G heads][64]
        const cuuint64_t dims[3] = {128, (cuuint64_t)n_heads, (cuuint64_t)n_rows};
        const cuuint64_t strides[2] = {128 * 2, (cuuint64_t)n_heads * 128 * 2};
        const cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(fp::ROWS / G)};
        const cuuint32_t elem[3] = {1, 1, 1};
        if (enc(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, elem,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return IB_ERR_UNSUPPORTED;
    }
    for (int which = 0; which < 2; ++which) {
        // pages [n_pages * n_kv_heads * page_size rows][128]: boxes of [page_size][64]
        const cuuint64_t dims[2] = {128, (cuuint64_t)n_pages * n_kv_heads * page_size};
        const cuuint64_t strides[1] = {128 * 2};
        const cuuint32_t box[2] = {64, (cuuint32_t)page_size};
        const cuuint32_t elem[2] = {1, 1};
        if (enc(which ? &mv : &mk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(which ? v_pages : k_pages), dims,
                strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return IB_ERR_UNSUPPORTED;
    }
    fp::Params P;
    P.block_table = block_table; P.tile_req = tile_req; P.tile_row0 = tile_row0; P.q_start = q_start;
    P.positions = positions; P.out = (__nv_bfloat16*)out; P.max_pages = max_pages; P.page_size = page_size;
    P.n_pages = n_pages; P.n_heads = n_heads; P.n_kv_heads = n_kv_heads; P.window = window;
    P.scale_log2 = scale * 1.4426950408889634f;
    const size_t smem = 2 * fp::TILE_BYTES + 4 * fp::TILE_BYTES + 20 * 8 + fp::SMEM_SLACK;
    static IbDeviceSet configured;   // the attribute is kept per device
    if (const int e = ib_allow_dynamic_smem(configured, fp::attention_pair_kernel, smem)) return e;
    ib_launch(fp::attention_pair_kernel, dim3(n_tiles * n_kv_heads), fp::THREADS, smem, stream, mq, mk, mv, P);
    return ib_launch_status();
}

// 0, or the code of the first bounded wait that ran out in the kernel above (1 producers, 2 to 4 the issuer, 5 and 6
// softmax).  Reading it synchronises with the device; `reset` clears it.
IB_EXPORT int ib_attention_pair_tcgen05_error(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, fp::g_error, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(fp::g_error, &zero, sizeof(int));
    }
    return v;
}

// The same word on its way to `out` (pinned host memory) in stream order, without waiting for the device: the
// caller reads it after an event that it records behind this call.
IB_EXPORT int ib_attention_pair_tcgen05_error_async(int* out, cudaStream_t stream) {
    return (int)cudaMemcpyFromSymbolAsync(out, fp::g_error, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
}

#else

IB_EXPORT int ib_paged_attention_pair_tcgen05(const void*, const void*, const void*, const int*, int, int, int, const int*,
                                              const int*, int, const int*, const int*, int, int, int, int, float, int, void*,
                                              cudaStream_t) {
    return IB_ERR_UNSUPPORTED;
}
IB_EXPORT int ib_attention_pair_tcgen05_error(int) { return 0; }

IB_EXPORT int ib_attention_pair_tcgen05_error_async(int* out, cudaStream_t) { *out = 0; return 0; }

#endif
