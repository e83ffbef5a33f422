// Paged grouped-query attention for prompt portions on tcgen05 tensor cores (bfloat16, head size 128).
//
// One CTA owns 128 query rows of one key/value head: 128/G consecutive tokens of one request with the G
// query heads that share the key/value head packed side by side (row = token * G + head).  Keys are
// walked in tiles of 128 (whole pages).  Per tile:
//   S  = Q K^T   one accumulator of 128 lanes x 128 columns in tensor memory (two of them, so that the
//                product for the next tile is issued while this tile's softmax runs),
//   P  = softmax step in registers: two threads per row (64 columns each) read the row of S with
//                tcgen05.ld, keep the running maximum and sum in float32 and write exp2(S - max) as bfloat16
//                into shared memory (two P tiles, used in turn),
//   PV = P V     two more accumulators, used in turn; the row's threads add a tile's product into their
//                float32 outputs one tile later, after rescaling them by the change of the maximum, so that
//                the product runs while the next tile's softmax is computed.
// Q, K and V arrive by TMA into 128-byte-swizzled tiles; K and V come page by page (a page of one head
// is a contiguous [page_size, 128] block) into a two-stage ring.  V is used as the MN-major operand of
// the second product, so no transposed copy of the cache is needed.
//
// Warps 0..7: softmax and output (warp w: lanes 32 (w % 4).., columns 64 (w / 4)..); warp 8: TMA producer of
// Q and K; warp 9: issuer of Q K^T and owner of the tensor-memory allocation; warp 10: TMA producer of V; warp
// 11: issuer of P V.  All mbarrier waits are bounded (about two seconds)
// and report through the library's error word.
#include <cuda.h>

#include "common.cuh"
#include "sm100.cuh"

#if IB_ACT_BF16

namespace fa {

using namespace sm100;

constexpr int D = 128;            // head size
constexpr int ROWS = 128;         // query rows per CTA
constexpr int KEYS = 128;         // keys per tile
constexpr int THREADS = 384;
constexpr int SMEM_SLACK = 512;   // bytes that the 1 KB alignment of the tiles may cost (the base is asked to be aligned)
constexpr int HALF_BYTES = 128 * 128;          // a [128 rows][64 elements] swizzled sub-tile
constexpr int TILE_BYTES = 2 * HALF_BYTES;     // Q, K, V or P tile: 128 x 128 bfloat16

__device__ int g_error = 0;

// a bounded wait that reports through this file's error word
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, int code) {
    return mbar_wait_bounded(bar, parity, &g_error, code);
}

// the two warps that share the rows 32 q .. 32 q + 31 (one per half of the columns) meet: barriers 2..5
__device__ __forceinline__ void pair_sync(int q) { asm volatile("bar.sync %0, 64;" ::"r"(2 + q) : "memory"); }

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

__global__ void __launch_bounds__(THREADS, 1) attention_kernel(const __grid_constant__ CUtensorMap map_q,
                                                               const __grid_constant__ CUtensorMap map_k,
                                                               const __grid_constant__ CUtensorMap map_v,
                                                               const Params P) {
    extern __shared__ __align__(1024) unsigned char raw_smem[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~(uintptr_t)1023);
    if (smem - raw_smem > SMEM_SLACK) {   // the tiles would not fit behind a base this far off a 1 KB boundary
        if (threadIdx.x == 0) atomicCAS(&g_error, 0, 9);
        return;
    }
    unsigned char* sq = smem;                       // Q tile
    unsigned char* sp = sq + TILE_BYTES;            // P tiles, used in turn
    unsigned char* sk = sp + 2 * TILE_BYTES;        // K tiles, two stages
    unsigned char* sv = sk + 2 * TILE_BYTES;        // V tiles, two stages
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(sv + 2 * TILE_BYTES);
    const unsigned q_full = smem_u32(bars), k_full0 = smem_u32(bars + 1), k_empty0 = smem_u32(bars + 3);
    const unsigned v_full0 = smem_u32(bars + 5), v_empty0 = smem_u32(bars + 7);
    const unsigned s_full0 = smem_u32(bars + 9), s_empty0 = smem_u32(bars + 11);
    const unsigned p_full0 = smem_u32(bars + 13), pv_full0 = smem_u32(bars + 15);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 17);
    float* xchg = reinterpret_cast<float*>(bars + 18);   // [2 in turn][2 halves][128 rows]: row maxima, later row sums

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
    const int tpt = ROWS / G;                       // tokens per tile (a group size that does not divide 128 leaves rows unused)
    int n_tok = P.q_start[req + 1] - row0;
    if (n_tok > tpt) n_tok = tpt;
    const int p0 = P.positions[row0];
    const int pmax = p0 + n_tok - 1;
    const int lo_min = (P.window > 0 && p0 - P.window + 1 > 0) ? p0 - P.window + 1 : 0;
    const int t_begin = lo_min / KEYS, t_end = pmax / KEYS + 1;   // key tiles
    const int n_tiles = t_end - t_begin;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(k_full0 + 8 * s, 1); mbar_init(k_empty0 + 8 * s, 1);
            mbar_init(v_full0 + 8 * s, 1); mbar_init(v_empty0 + 8 * s, 1);
            mbar_init(s_full0 + 8 * s, 1); mbar_init(s_empty0 + 8 * s, 8);
            mbar_init(p_full0 + 8 * s, 8); mbar_init(pv_full0 + 8 * s, 1);
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
    const unsigned tmem = *tmem_slot;      // columns 0..127 S0, 128..255 S1, 256..383 PV0, 384..511 PV1
    bool ok = true;

    if (warp == 8 || warp == 10) {
        // TMA producers: warp 8 brings the queries and the key tiles, warp 10 the value tiles.  Lane p brings page
        // p of every tile (two boxes: the 64-column halves) and looks the page up one tile ahead of its use.
        if (warp == 8 && lane == 0) {
            mbar_expect_tx(q_full, tpt * G * 256);   // [tokens][G heads][128] as two 64-column halves (rows beyond tokens x G stay unwritten: no row reads another)
            tma_load_3d(smem_u32(sq), &map_q, 0, kvh * G, row0, q_full);
            tma_load_3d(smem_u32(sq + HALF_BYTES), &map_q, 64, kvh * G, row0, q_full);
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
        auto load_tile = [&](int i, int page, bool keys) {
            const int s = i & 1;
            const unsigned full = (keys ? k_full0 : v_full0) + 8 * s;
            if (lane == 0) mbar_expect_tx(full, TILE_BYTES);
            __syncwarp();
            if (lane < pages_per_tile) {
                const int grow = (page * P.n_kv_heads + kvh) * P.page_size;
                const unsigned off = (unsigned)(lane * P.page_size) * 128u;
                unsigned char* dst = (keys ? sk : sv) + s * TILE_BYTES;
                tma_load_2d(smem_u32(dst) + off, keys ? &map_k : &map_v, 0, grow, full);
                tma_load_2d(smem_u32(dst + HALF_BYTES) + off, keys ? &map_k : &map_v, 64, grow, full);
            }
        };
        // The key tiles and the value tiles are asked for by a warp each: asking for a tile is sixteen pages of
        // two boxes, about as long as the products of a tile take.  Keys run a tile ahead: K(i) is free again as
        // soon as the scores of tile i - 2 are done, V(i) only after the second product of tile i - 2.
        const bool keys = warp == 8;
        const unsigned empty0 = keys ? k_empty0 : v_empty0;
        int page = n_tiles > 0 ? lookup(0) : 0;
        for (int i = 0; i < n_tiles; ++i) {
            const int page_next = i + 1 < n_tiles ? lookup(i + 1) : 0;
            if (i >= 2 && ok && !mbar_wait(empty0 + 8 * (i & 1), ((i >> 1) - 1) & 1, 1)) ok = false;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            load_tile(i, page, keys);
            page = page_next;
        }
    } else if (warp == 9 || warp == 11) {
        // The two products of a tile are issued by a thread each (warp 9: S = Q K^T, warp 11: P V): a thread that
        // issues is held at the pace of the tensor pipe, and every wait on a barrier costs it a few hundred
        // cycles; one thread for both left the pipe idle two thirds of the time.
        // Both products: M = 128, N = 128, bfloat16 in, float32 out; the second takes V as MN-major B.
        const unsigned idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(KEYS >> 3) << 17) | ((unsigned)(ROWS >> 4) << 24);
        const unsigned idesc_pv = idesc_qk | (1u << 16);
        if (warp == 9 && lane == 0) {
            for (int i = 0; i < n_tiles; ++i) {   // S(i) = Q K(i)^T into buffer i & 1, a tile ahead of its softmax
                const int s = i & 1;
                if (i == 0 && !mbar_wait(q_full, 0, 2)) { ok = false; break; }
                if (!mbar_wait(k_full0 + 8 * s, (i >> 1) & 1, 2)) { ok = false; break; }
                if (i >= 2 && !mbar_wait(s_empty0 + 8 * s, ((i >> 1) - 1) & 1, 3)) { ok = false; break; }
                fence_after();
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const unsigned off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
                    umma(tmem + s * 128, desc_k_major(smem_u32(sq) + off), desc_k_major(smem_u32(sk + s * TILE_BYTES) + off),
                         idesc_qk, k != 0);
                }
                umma_commit(s_full0 + 8 * s);
                umma_commit(k_empty0 + 8 * s);   // K(i) is free once these products are done
            }
        } else if (warp == 11 && lane == 0) {
            for (int i = 0; i < n_tiles; ++i) {
                const int s = i & 1;
                if (!mbar_wait(p_full0 + 8 * s, (i >> 1) & 1, 4)) { ok = false; break; }
                if (!mbar_wait(v_full0 + 8 * s, (i >> 1) & 1, 2)) { ok = false; break; }
                fence_after();
#pragma unroll
                for (int k = 0; k < KEYS / 16; ++k) {
                    const unsigned aoff = (k >> 2) * HALF_BYTES + (k & 3) * 32;   // P: K-major, 16 keys = 32 bytes
                    const unsigned boff = k * 16 * 128;                            // V: 16 key rows further
                    umma(tmem + 256 + s * 128, desc_k_major(smem_u32(sp + s * TILE_BYTES) + aoff),
                         desc_mn_major(smem_u32(sv + s * TILE_BYTES) + boff, HALF_BYTES), idesc_pv, k != 0);
                }
                umma_commit(pv_full0 + 8 * s);
                umma_commit(v_empty0 + 8 * s);    // V(i) is free once these products are done
            }
        }
    } else if (warp < 8) {
        // softmax and output: two threads per row of the tile; this one has columns 64 * ch .. 64 * ch + 63
        const int ch = warp >> 2;
        const int r = (warp & 3) * 32 + lane;
        const int ti = r / G, g = r - ti * G;
        const bool row_valid = ti < n_tok;
        const int pos = row_valid ? p0 + ti : -1;
        const int lo = (row_valid && P.window > 0 && pos - P.window + 1 > 0) ? pos - P.window + 1 : 0;
        float o[64];
#pragma unroll
        for (int e = 0; e < 64; ++e) o[e] = 0.0f;
        float m = -INFINITY, l = 0.0f, corr_pending = 1.0f;
        const unsigned lane_addr = (unsigned)((warp & 3) * 32) << 16;
        auto add_product = [&](int i, float corr) {   // o = o * corr + (P V)(i), this thread's 64 columns
            unsigned a[32], b[32];
            tmem_ld32_issue(tmem + lane_addr + 256 + (i & 1) * 128 + ch * 64, a);
            tmem_ld32_issue(tmem + lane_addr + 256 + (i & 1) * 128 + ch * 64 + 32, b);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                o[j] = o[j] * corr + __uint_as_float(a[j]);
                o[32 + j] = o[32 + j] * corr + __uint_as_float(b[j]);
            }
        };
        // After a wait has run out the loop goes on without waiting, so that every thread still meets its
        // partner at the named barrier the same number of times; the output is not stored then.
        for (int i = 0; i < n_tiles; ++i) {
            const int s = i & 1;
            if (ok && !mbar_wait(s_full0 + 8 * s, (i >> 1) & 1, 5)) ok = false;
            fence_after();
            const int key0 = (t_begin + i) * KEYS + ch * 64;
            unsigned a[32], b[32];
            tmem_ld32_issue(tmem + lane_addr + s * 128 + ch * 64, a);
            tmem_ld32_issue(tmem + lane_addr + s * 128 + ch * 64 + 32, b);
            tmem_ld_wait();
            // a tile whose 64 keys this row sees in full needs no comparisons (all tiles but the first and last few)
            const bool all_visible = key0 >= lo && key0 + 63 <= pos;
            // (four running maxima, and four running sums below: one chain of 64 dependent operations would
            // leave the two warps of a scheduler waiting on each other's latencies)
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
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // the row's maximum over both halves (raw scores; the scale is positive)
            // (two exchange buffers in turn: the partner has read buffer i & 1 before it can arrive at the next
            // tile's barrier, which this thread passes before it writes that buffer again two tiles on)
            float* xb = xchg + (i & 1) * 256;
            xb[ch * 128 + r] = mx;
            pair_sync(warp & 3);
            mx = fmaxf(mx, xb[(ch ^ 1) * 128 + r]) * P.scale_log2;
            const float m_new = fmaxf(m, mx);
            const float m_safe = m_new == -INFINITY ? 0.0f : m_new;
            const float corr = m == -INFINITY ? 0.0f : ex2(m - m_safe);
            float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            unsigned char* prow = sp + s * TILE_BYTES + ch * HALF_BYTES + r * 128;
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
            l = l * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            m = m_new;
            // S(i) has been read and P(i) written: tell the MMA issuer (one arrival per warp)
            fence_before();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> the tensor core's reads
            __syncwarp();
            if (lane == 0) { mbar_arrive(s_empty0 + 8 * s); mbar_arrive(p_full0 + 8 * s); }
            // the product of the tile before this one has had this tile's softmax to finish
            if (i > 0) {
                if (ok && !mbar_wait(pv_full0 + 8 * ((i - 1) & 1), ((i - 1) >> 1) & 1, 6)) ok = false;
                fence_after();
                add_product(i - 1, corr_pending);
                fence_before();
            }
            corr_pending = corr;
        }
        if (ok && n_tiles > 0) {
            const int i = n_tiles - 1;
            if (mbar_wait(pv_full0 + 8 * (i & 1), (i >> 1) & 1, 6)) {
                fence_after();
                add_product(i, corr_pending);
                fence_before();
            } else {
                ok = false;
            }
        }
        // the row's sum over both halves
        float* xb = xchg + (n_tiles & 1) * 256;
        xb[ch * 128 + r] = l;
        pair_sync(warp & 3);
        l += xb[(ch ^ 1) * 128 + r];
        if (row_valid && ok) {
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            __nv_bfloat16* dst = P.out + ((long)(row0 + ti) * P.n_heads + kvh * G + g) * D + ch * 64;
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 8) {
                uint4 w;
                w.x = pack_bf16(o[c0] * inv, o[c0 + 1] * inv); w.y = pack_bf16(o[c0 + 2] * inv, o[c0 + 3] * inv);
                w.z = pack_bf16(o[c0 + 4] * inv, o[c0 + 5] * inv); w.w = pack_bf16(o[c0 + 6] * inv, o[c0 + 7] * inv);
                *reinterpret_cast<uint4*>(dst + c0) = w;
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

}  // namespace fa

// Prefill-form attention for head size 128, bfloat16: tile i holds up to 128/G tokens of request tile_req[i]
// from row tile_row0[i].  Same arguments and results as ib_paged_attention_mma with decode_form = 0.
IB_EXPORT int ib_paged_attention_tcgen05(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                         int max_pages, int page_size, int n_pages, const int* tile_req,
                                         const int* tile_row0, int n_tiles, const int* q_start, const int* positions,
                                         int n_rows, int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                                         void* out, cudaStream_t stream) {
    if (n_tiles <= 0) return IB_OK;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads || page_size <= 0 || max_pages <= 0) return IB_ERR_ARGUMENT;
    const int G = n_heads / n_kv_heads;
    if (head_dim != fa::D || fa::KEYS % page_size || page_size < 8 || G > fa::ROWS) return IB_ERR_UNSUPPORTED;
    if (!(scale > 0.0f)) return IB_ERR_UNSUPPORTED;   // the row maximum is taken before the scale is applied
    fa::EncodeTiled enc = fa::encode_fn();
    if (enc == nullptr) return IB_ERR_UNSUPPORTED;
    CUtensorMap mq, mk, mv;
    {
        // q [n_rows tokens][n_heads][128]: boxes of [128/G tokens][G heads][64]
        const cuuint64_t dims[3] = {128, (cuuint64_t)n_heads, (cuuint64_t)n_rows};
        const cuuint64_t strides[2] = {128 * 2, (cuuint64_t)n_heads * 128 * 2};
        const cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(fa::ROWS / G)};
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
    fa::Params P;
    P.block_table = block_table; P.tile_req = tile_req; P.tile_row0 = tile_row0; P.q_start = q_start;
    P.positions = positions; P.out = (__nv_bfloat16*)out; P.max_pages = max_pages; P.page_size = page_size;
    P.n_pages = n_pages; P.n_heads = n_heads; P.n_kv_heads = n_kv_heads; P.window = window;
    P.scale_log2 = scale * 1.4426950408889634f;
    const size_t smem = 7 * fa::TILE_BYTES + 18 * 8 + 4 * 128 * 4 + fa::SMEM_SLACK;
    static IbDeviceSet configured;   // the attribute is kept per device
    if (const int e = ib_allow_dynamic_smem(configured, fa::attention_kernel, smem)) return e;
    ib_launch(fa::attention_kernel, dim3(n_tiles * n_kv_heads), fa::THREADS, smem, stream, mq, mk, mv, P);
    return ib_launch_status();
}

IB_EXPORT int ib_attention_tcgen05_error(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, fa::g_error, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(fa::g_error, &zero, sizeof(int));
    }
    return v;
}

// The same word on its way to `out` (pinned host memory) in stream order, without waiting for the device: the
// caller reads it after an event that it records behind this call.
IB_EXPORT int ib_attention_tcgen05_error_async(int* out, cudaStream_t stream) {
    return (int)cudaMemcpyFromSymbolAsync(out, fa::g_error, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
}

#else  // the float32 build has no tensor-core attention

IB_EXPORT int ib_paged_attention_tcgen05(const void*, const void*, const void*, const int*, int, int, int, const int*,
                                         const int*, int, const int*, const int*, int, int, int, int, float, int, void*,
                                         cudaStream_t) {
    return IB_ERR_UNSUPPORTED;
}

IB_EXPORT int ib_attention_tcgen05_error(int) { return 0; }

IB_EXPORT int ib_attention_tcgen05_error_async(int* out, cudaStream_t) { *out = 0; return 0; }

#endif
