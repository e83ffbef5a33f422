// Paged grouped-query attention for prompt portions on tcgen05 tensor cores (bfloat16, head size 128): two query
// tiles per CTA that take turns.
//
// One CTA owns 256 query rows of one key/value head as two tiles of 128 rows: tile t holds 128/G consecutive
// tokens of one request with the G query heads that share the key/value head side by side (row = token * G +
// head); tile 1 continues where tile 0 ends.  Keys are walked in tiles of 64 (whole pages), and every key and
// value tile that arrives serves both query tiles.  Per key tile and query tile:
//   S  = Q K^T   128 lanes x 64 columns in tensor memory, two buffers per query tile in turn;
//   P  = exp2(S * scale - m) by ONE thread per row: it reads its row of S with tcgen05.ld, keeps the running
//        reference maximum m and the sum in float32 and writes P as bfloat16 into shared memory (two P tiles per
//        query tile in turn);
//   O += P V     accumulated in tensor memory over all key tiles (128 lanes x 128 columns per query tile) and read
//        once at the end.  The reference maximum of a row moves only when the row's maximum has grown by more than
//        8 (a factor of 256) since it was set; then the row of O and the sum are scaled to the new reference first.
//        Until then P may reach 256, which bfloat16 and the float32 sums hold as well as values below 1, so the
//        result is the same softmax.
// While one query tile's threads are busy with exponentials, the other's read, compare and write, and the
// tensor pipe works for whichever is ready.
//
// Warps 0..3: softmax and output of query tile 0 (warp w: lanes 32 w ..); warps 4..7: of query tile 1; warp 8:
// TMA producer of Q and K; warp 9: issuer of Q K^T and owner of the tensor-memory allocation; warp 10: TMA
// producer of V; warp 11: issuer of P V.  All mbarrier waits are bounded (about two seconds) and report through
// the library's error word.
#include <cuda.h>

#include "common.cuh"
#include "sm100.cuh"

#if IB_ACT_BF16

namespace fp {

using namespace sm100;

constexpr int D = 128;                 // head size
constexpr int ROWS = 128;              // rows of a query tile
constexpr int KEYS = 64;               // keys per tile
constexpr int THREADS = 384;
constexpr int SMEM_SLACK = 1024;       // bytes that the 1 KB alignment of the tiles may cost
constexpr int Q_HALF = ROWS * 128;     // [128 rows][64 elements] swizzled sub-tile of Q
constexpr int Q_TILE = 2 * Q_HALF;
constexpr int KV_HALF = KEYS * 128;    // [64 keys][64 elements] swizzled sub-tile of K or V
constexpr int KV_TILE = 2 * KV_HALF;
constexpr int P_TILE = ROWS * 128;     // [128 rows][64 keys]
constexpr float RESCALE_STEP = 8.0f;   // how far a row's maximum may outgrow its reference (in powers of two)

__device__ int g_error = 0;

// a bounded wait that reports through this file's error word
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, int code) {
    return mbar_wait_bounded(bar, parity, &g_error, code);
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
    unsigned char* sp = sq + 2 * Q_TILE;            // P tiles: [query tile][buffer]
    unsigned char* sk = sp + 4 * P_TILE;            // K tiles, two stages
    unsigned char* sv = sk + 2 * KV_TILE;           // V tiles, two stages
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(sv + 2 * KV_TILE);
    const unsigned q_full = smem_u32(bars);
    const unsigned k_full0 = smem_u32(bars + 1), k_empty0 = smem_u32(bars + 3);
    const unsigned v_full0 = smem_u32(bars + 5), v_empty0 = smem_u32(bars + 7);
    // per query tile t and buffer b: index 2 t + b
    const unsigned s_full0 = smem_u32(bars + 9), s_empty0 = smem_u32(bars + 13);
    const unsigned p_full0 = smem_u32(bars + 17), p_empty0 = smem_u32(bars + 21);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 25);

    ib_grid_dependency_sync();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the last tiles of a prompt see the most keys: they are started first, so that the grid's tail is short
    const int tile = gridDim.x - 1 - blockIdx.x, kvh = blockIdx.y;
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
        }
        for (int s = 0; s < 4; ++s) {
            mbar_init(s_full0 + 8 * s, 1); mbar_init(s_empty0 + 8 * s, 4);
            mbar_init(p_full0 + 8 * s, 4); mbar_init(p_empty0 + 8 * s, 1);
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
    const unsigned tmem = *tmem_slot;      // columns 64 (2 t + b): S of query tile t, buffer b; 256 + 128 t: O of tile t
    bool ok = true;

    if (warp == 8 || warp == 10) {
        // TMA producers: warp 8 brings the queries and the key tiles, warp 10 the value tiles.  Lane p brings page
        // p of every tile (two boxes: the 64-column halves) and looks the page up one tile ahead of its use.
        if (warp == 8 && lane == 0) {
            const int n_q = n_tok_t[1] > 0 ? 2 : 1;
            mbar_expect_tx(q_full, n_q * tpt * G * 256);   // per tile [tokens][G heads][128] as two 64-column halves
            for (int t = 0; t < n_q; ++t) {
                tma_load_3d(smem_u32(sq + t * Q_TILE), &map_q, 0, kvh * G, row0 + t * tpt, q_full);
                tma_load_3d(smem_u32(sq + t * Q_TILE + Q_HALF), &map_q, 64, kvh * G, row0 + t * tpt, q_full);
            }
        }
        const int* bt = P.block_table + (long)req * P.max_pages;
        const int pages_per_tile = KEYS / P.page_size;   // at most 8
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
            if (lane == 0) mbar_expect_tx(full0 + 8 * s, KV_TILE);
            __syncwarp();
            if (lane < pages_per_tile) {
                const int grow = (page * P.n_kv_heads + kvh) * P.page_size;
                const unsigned off = (unsigned)(lane * P.page_size) * 128u;
                unsigned char* dst = (keys ? sk : sv) + s * KV_TILE;
                tma_load_2d(smem_u32(dst) + off, keys ? &map_k : &map_v, 0, grow, full0 + 8 * s);
                tma_load_2d(smem_u32(dst + KV_HALF) + off, keys ? &map_k : &map_v, 64, grow, full0 + 8 * s);
            }
            page = page_next;
        }
    } else if (warp == 9 || warp == 11) {
        // S = Q K^T: M = 128, N = 64; O += P V: M = 128, N = 128 with V as MN-major B; bfloat16 in, float32 out
        const unsigned idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(KEYS >> 3) << 17) | ((unsigned)(ROWS >> 4) << 24);
        const unsigned idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(D >> 3) << 17) | ((unsigned)(ROWS >> 4) << 24);
        if (warp == 9 && lane == 0) {
            if (n_tiles > 0 && !mbar_wait(q_full, 0, 2)) ok = false;
            for (int i = 0; i < n_tiles && ok; ++i) {
                const int s = i & 1;
                if (!mbar_wait(k_full0 + 8 * s, (i >> 1) & 1, 2)) { ok = false; break; }
                for (int t = 0; t < 2 && ok; ++t) {
                    if (i >= n_tiles_t[t]) continue;
                    const int sb = 2 * t + s;
                    if (i >= 2 && !mbar_wait(s_empty0 + 8 * sb, ((i >> 1) - 1) & 1, 3)) { ok = false; break; }
                    fence_after();
#pragma unroll
                    for (int k = 0; k < D / 16; ++k) {
                        const unsigned qoff = (k >> 2) * Q_HALF + (k & 3) * 32, koff = (k >> 2) * KV_HALF + (k & 3) * 32;
                        umma(tmem + sb * 64, desc_k_major(smem_u32(sq + t * Q_TILE) + qoff),
                             desc_k_major(smem_u32(sk + s * KV_TILE) + koff), idesc_qk, k != 0);
                    }
                    umma_commit(s_full0 + 8 * sb);
                }
                umma_commit(k_empty0 + 8 * s);   // K(i) is free once these products are done
            }
        } else if (warp == 11 && lane == 0) {
            for (int i = 0; i < n_tiles && ok; ++i) {
                const int s = i & 1;
                if (!mbar_wait(v_full0 + 8 * s, (i >> 1) & 1, 2)) { ok = false; break; }
                for (int t = 0; t < 2 && ok; ++t) {
                    if (i >= n_tiles_t[t]) continue;
                    const int sb = 2 * t + s;
                    if (!mbar_wait(p_full0 + 8 * sb, (i >> 1) & 1, 4)) { ok = false; break; }
                    fence_after();
#pragma unroll
                    for (int k = 0; k < KEYS / 16; ++k)   // P: K-major, 16 keys = 32 bytes; V: 16 key rows further
                        umma(tmem + 256 + t * 128, desc_k_major(smem_u32(sp + sb * P_TILE) + k * 32),
                             desc_mn_major(smem_u32(sv + s * KV_TILE) + k * 16 * 128, KV_HALF), idesc_pv, (i | k) != 0);
                    umma_commit(p_empty0 + 8 * sb);   // P(i) is free, and O holds tile i, once these products are done
                }
                umma_commit(v_empty0 + 8 * s);        // V(i) is free once these products are done
            }
        }
    } else {
        // softmax and output: one thread per row of its query tile
        const int t = warp >> 2;
        const int r = (warp & 3) * 32 + lane;
        const int ti = r / G, g = r - ti * G;
        const bool row_valid = ti < n_tok_t[t];
        const int pos = row_valid ? p0 + t * tpt + ti : -1;
        const int lo = (row_valid && P.window > 0 && pos - P.window + 1 > 0) ? pos - P.window + 1 : 0;
        const unsigned lane_addr = (unsigned)((warp & 3) * 32) << 16;
        const unsigned o_addr = tmem + lane_addr + 256 + t * 128;
        float m_ref = -INFINITY, l = 0.0f;   // the reference that P and O are scaled to, and the sum of P
        const int my_tiles = n_tiles_t[t];
        for (int i = 0; i < my_tiles; ++i) {
            const int sb = 2 * t + (i & 1);
            if (ok && !mbar_wait(s_full0 + 8 * sb, (i >> 1) & 1, 5)) ok = false;
            ok = __all_sync(0xffffffffu, ok);   // the tensor-memory loads and stores below are warp-wide
            if (!ok) break;
            fence_after();
            const int key0 = (t_begin + i) * KEYS;
            unsigned a[32], b[32];
            tmem_ld32_issue(tmem + lane_addr + sb * 64, a);
            tmem_ld32_issue(tmem + lane_addr + sb * 64 + 32, b);
            tmem_ld_wait();
            // S(i) is in registers: its buffer may take the tile after next
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_empty0 + 8 * sb);
            // a tile whose 64 keys this row sees in full needs no comparisons (all tiles but the first and last few)
            const bool all_visible = key0 >= lo && key0 + 63 <= pos;
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (all_visible) {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    mx4[j & 3] = fmaxf(mx4[j & 3], fmaxf(__uint_as_float(a[j]), __uint_as_float(b[j])));
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int ka = key0 + j, kb = key0 + 32 + j;
                    if (!(ka >= lo && ka <= pos)) a[j] = 0xff800000u;   // -inf
                    if (!(kb >= lo && kb <= pos)) b[j] = 0xff800000u;
                    mx4[j & 3] = fmaxf(mx4[j & 3], fmaxf(__uint_as_float(a[j]), __uint_as_float(b[j])));
                }
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * P.scale_log2;   // the scale is positive
            // Move the reference?  Only if the maximum has outgrown it by more than the step (or there is none yet).
            const bool move = mx > m_ref + RESCALE_STEP || (m_ref == -INFINITY && mx > -INFINITY);
            if (i > 0 && __any_sync(0xffffffffu, move)) {
                // O holds the tiles up to i - 1 once their products are done; scale this warp's rows of it
                const int pb = 2 * t + ((i - 1) & 1);
                if (!mbar_wait(p_empty0 + 8 * pb, ((i - 1) >> 1) & 1, 6)) ok = false;
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
                tmem_st_wait();
                l *= corr;
            }
            if (move) m_ref = mx;
            const float m_safe = m_ref == -INFINITY ? 0.0f : m_ref;
            // the P tile that this row is written to must have been read by the product two tiles back
            if (i >= 2) {
                if (!mbar_wait(p_empty0 + 8 * sb, ((i >> 1) - 1) & 1, 7)) ok = false;
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            unsigned char* prow = sp + sb * P_TILE + r * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                float p[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int e = 8 * c + j;
                    const float x = __uint_as_float(e < 32 ? a[e] : b[e - 32]);
                    p[j] = ex2(fmaf(x, P.scale_log2, -m_safe));   // exp2(-inf) = 0 for keys that are not seen
                    sum4[j & 3] += p[j];
                }
                uint4 w;
                w.x = pack_bf16(p[0], p[1]); w.y = pack_bf16(p[2], p[3]);
                w.z = pack_bf16(p[4], p[5]); w.w = pack_bf16(p[6], p[7]);
                *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = w;
            }
            l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            // P(i) is written (and O scaled, if it was): tell the issuer of P V (one arrival per warp)
            fence_before();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> the tensor core's reads
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full0 + 8 * sb);
        }
        if (ok && my_tiles > 0) {
            const int i = my_tiles - 1;
            if (!mbar_wait(p_empty0 + 8 * (2 * t + (i & 1)), (i >> 1) & 1, 6)) ok = false;
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
    const size_t smem = 2 * fp::Q_TILE + 4 * fp::P_TILE + 4 * fp::KV_TILE + 26 * 8 + fp::SMEM_SLACK;
    static IbDeviceSet configured;   // the attribute is kept per device
    if (const int e = ib_allow_dynamic_smem(configured, fp::attention_pair_kernel, smem)) return e;
    ib_launch(fp::attention_pair_kernel, dim3(n_tiles, n_kv_heads), fp::THREADS, smem, stream, mq, mk, mv, P);
    return ib_launch_status();
}

// 0, or the code of the first bounded wait that ran out in the kernel above (1 producer, 2 to 4 issuers, 5 to 7
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
