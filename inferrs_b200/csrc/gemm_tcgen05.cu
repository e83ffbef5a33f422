// y[t, f] = sum_k x[t, k] * w[f, k]  on the fifth-generation tensor cores (bfloat16 in, float32 accumulate).
//
// The weight matrix is the 128-row operand of tcgen05.mma and the tokens are its N dimension
// (16..256 per tile), so a decode step with a handful of tokens still issues full-height MMAs and the
// kernel's work is streaming W through shared memory: TMA brings 128x64 tiles of W and BNx64 tiles of x
// into a ring of 128-byte-swizzled stages, one thread issues the MMAs, the accumulator (128 lanes x BN
// columns of float32) lives in tensor memory, and four warps read it back with tcgen05.ld and store
// y.  Roles: warp 0 = TMA producer, warp 1 = MMA issuer and owner of the tensor-memory allocation,
// warps 2..5 = epilogue (one quarter of the 128 lanes each).
//
// With few output tiles the K range is cut over a thread-block cluster (1,1,split): every CTA of the
// cluster accumulates its part of K and the parts are summed through distributed shared memory, so no
// global scratch and no atomics are needed.  Up to 32 tokens every CTA of the cluster owns an equal share
// of the tile's rows: each CTA stores the other shares of its partial sums straight into their owners'
// shared memory, one cluster barrier follows, and every owner adds the parts in the order of the CTAs'
// ranks and stores its rows.  Wider tiles are summed by the cluster's first CTA, which reads the others.
//
// Two things can be folded into the read-back of up to 32 tokens, so that the norm between two products needs no
// kernel of its own (x / sqrt(mean(x^2) + eps) * w is the same as (x * w) scaled by the row's 1 / sqrt(...)):
//   * the residual stream: y is added to a float32 stream in place, the stream times the weight vector of the norm
//     that follows is stored as bfloat16 instead of y, and every CTA writes the sums of squares of its share of
//     the stream's rows to a list of parts ("sink");
//   * the row scale: x is such a stream-times-weight matrix with its list of parts; the parts are added up in a
//     fixed order while the weights stream in, and the accumulator is scaled by 1 / sqrt(sum / width + eps) per
//     token before it is used ("scaled rows").
//
// A tile may cover fewer rows of W than the MMA's 128 (the TMA box is lower; the accumulator's other rows are never
// stored): the host lowers the tiles of a product whose CTAs number between one and two per SM until every SM has
// two, because such a product ends when its fullest SM does (see tile_rows_for).
//
// Every wait on an mbarrier is bounded (about two seconds); a wait that runs out records a code in the
// library's error word, the CTA lets outstanding copies land, frees its tensor memory and returns.
#include <cuda.h>

#include "common.cuh"
#include "sm100.cuh"

#if IB_ACT_BF16

namespace tc {

using namespace sm100;

constexpr int BM = 128;       // rows of W per tile (MMA M)
constexpr int BK = 64;        // K per stage: 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int A_BYTES = BM * BK * 2;

__device__ int g_error = 0;   // 0 ok; else (role code) of the first wait that ran out

// a bounded wait that reports through this file's error word
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, int code) {
    return mbar_wait_bounded(bar, parity, &g_error, code);
}
static int g_pdl = 0;          // host: launch with programmatic stream serialization (see ib_gemm_tcgen05_set_pdl)

__device__ __forceinline__ void cluster_sync_all() {
    __syncwarp();  // lanes that skipped a single-lane role loop join the others before the aligned barrier
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_arrive() {
    __syncwarp();
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
    __syncwarp();
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ float ld_remote_f32(unsigned local_addr, unsigned rank) {
    unsigned remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

__device__ __forceinline__ void st_remote_f32(unsigned local_addr, unsigned rank, float v) {
    unsigned remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

struct Params {
    void* y;
    long ldy;
    int n_tok, n_out, num_kb, y_is_f32;
    int inner;   // gated form: rows of the gate matrix; the up matrix follows it in w
    int tile_rows;   // rows of W that a tile covers (gated form: of each of the two matrices); the MMA's other rows are not used
    // scaled rows (null: x is used as it is): parts of the sums of squares of x's rows [n_in_parts][SSQ_LD]
    const float* in_ssq;
    int n_in_parts;
    float in_eps, in_inv_width;
    // sink (null: y is stored as it is): the float32 stream [n_tok, n_out] that y is added to, the weight vector
    // [n_out] that the stream is multiplied by before it is stored in y's place, and where this CTA's part of the
    // rows' sums of squares goes: [tiles * splits][SSQ_LD]
    float* residual;
    long ld_res;
    const void* sink_w;
    int sink_w_is_f32;
    float* out_ssq;
};

constexpr int SSQ_LD = 32;    // tokens per part of a list of sums of squares (the folded forms take up to 32 tokens)

// What the read-back does with one finished value: scale it by its token's row scale, then either hand it on as it
// is or add it to the stream (rounded to bfloat16 first, as it is when the product stores it and a norm kernel adds
// it) and hand on the stream times the norm's weight.  `ssq` gathers the squares of the stream's new values.  The
// stream's old value and the weight were fetched while the weights streamed in.
__device__ __forceinline__ float finish_value(const Params& p, float v, int tok, int feature, float inv, float old,
                                              float w, float& ssq) {
    v *= inv;
    if (p.residual == nullptr) return v;
    const float s = old + __bfloat162float(__float2bfloat16_rn(v));
    p.residual[(long)tok * p.ld_res + feature] = s;
    ssq += s * s;
    return s * w;
}
__device__ __forceinline__ float sink_weight(const Params& p, int feature) {
    return p.sink_w_is_f32 ? reinterpret_cast<const float*>(p.sink_w)[feature]
                           : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.sink_w)[feature]);
}

template <int BN, int STAGES, int MODE>
__global__ void __launch_bounds__(THREADS, (BN <= 64 ? 2 : 1)) gemm_kernel(const __grid_constant__ CUtensorMap map_w,
                                                          const __grid_constant__ CUtensorMap map_x, const Params p) {
    constexpr int B_BYTES = BN * BK * 2;
    constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    constexpr bool SCATTER = BN <= 32;   // how a cluster sums its parts: see the head of this file
    extern __shared__ unsigned char raw_smem[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~(uintptr_t)1023);
    unsigned char* a_tiles = smem;
    unsigned char* b_tiles = smem + STAGES * A_BYTES;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(b_tiles + STAGES * B_BYTES);
    const unsigned full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES), accum = smem_u32(bars + 2 * STAGES);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * STAGES + 1);
    float* fold = reinterpret_cast<float*>(bars + 2 * STAGES + 2);   // [8][32] partial sums, then [32] row scales (folded forms)
    float* recv = fold + 9 * SSQ_LD;                                  // [rank of the sender][BN][rows owned], SCATTER only

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_f = blockIdx.x, tile_t = blockIdx.y;
    const int splits = gridDim.z;
    const int kb_per = (p.num_kb + splits - 1) / splits;
    const int kb0 = blockIdx.z * kb_per;
    const int nkb = (kb0 + kb_per <= p.num_kb ? kb_per : p.num_kb - kb0);  // >= 1: the host keeps splits <= num_kb / 1

    // Under programmatic dependent launch the next kernel of the stream may start its own prologue now; this
    // kernel in turn may have been started before its predecessor finished, so it reads the weights (which no
    // kernel writes) at once but touches x, y and the rest only after griddepcontrol.wait.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before();
    __syncthreads();
    fence_after();
    const unsigned tmem = *tmem_slot;
    bool ok = true;
    // A CTA's shared memory may be written by its cluster only once the CTA runs: every CTA says so here and
    // looks at the others' word just before its first store to them, long after they have given it.
    if (splits > 1 && SCATTER) cluster_arrive();

    if (warp == 0) {
        if (lane == 0 && nkb > 0) {
            // the weights are read once: their lines are the first to leave the L2 cache again
            const unsigned long long pol = policy_evict_first();
            // what a stage receives: the boxes of W are tile_rows high, whatever the MMA's height
            const unsigned stage_bytes = (unsigned)((MODE == 1 ? 2 : 1) * p.tile_rows * BK * 2 + B_BYTES);
            auto load_w = [&](int i, int s) {   // k-block i of this CTA's part into stage s
                const unsigned dst = smem_u32(a_tiles + s * A_BYTES);
                if (MODE == 1) {   // up to 64 rows of the gate matrix, and the same rows of the up matrix 64 rows below them in the stage
                    tma_load_2d_hint(dst, &map_w, (kb0 + i) * BK, tile_f * p.tile_rows, full0 + 8 * s, pol);
                    tma_load_2d_hint(dst + A_BYTES / 2, &map_w, (kb0 + i) * BK, p.inner + tile_f * p.tile_rows, full0 + 8 * s, pol);
                } else {
                    tma_load_2d_hint(dst, &map_w, (kb0 + i) * BK, tile_f * p.tile_rows, full0 + 8 * s, pol);
                }
            };
            // the first ring of weight tiles is on its way before the predecessor's results are waited for
            const int head = nkb < STAGES ? nkb : STAGES;
            for (int i = 0; i < head; ++i) {
                mbar_expect_tx(full0 + 8 * i, stage_bytes);
                load_w(i, i);
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int i = 0; i < head; ++i)
                tma_load_2d(smem_u32(b_tiles + i * B_BYTES), &map_x, (kb0 + i) * BK, tile_t * BN, full0 + 8 * i);
            for (int i = head; i < nkb; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(empty0 + 8 * s, ((i / STAGES) - 1) & 1, 1)) { ok = false; break; }
                mbar_expect_tx(full0 + 8 * s, stage_bytes);
                load_w(i, s);
                tma_load_2d(smem_u32(b_tiles + s * B_BYTES), &map_x, (kb0 + i) * BK, tile_t * BN, full0 + 8 * s);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(full0 + 8 * s, (i / STAGES) & 1, 2)) { ok = false; break; }
                fence_after();
                const unsigned long long da = desc_k_major(smem_u32(a_tiles + s * A_BYTES));
                const unsigned long long db = desc_k_major(smem_u32(b_tiles + s * B_BYTES));
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    umma(tmem, da + (unsigned long long)(k * UMMA_K * 2 / 16), db + (unsigned long long)(k * UMMA_K * 2 / 16),
                         idesc, (i | k) != 0);
                umma_commit(empty0 + 8 * s);   // arrives when these MMAs have read the stage
            }
            umma_commit(accum);                // arrives when every MMA above has written the accumulator
        }
    }

    const int q = warp & 3;                    // the quarter of the 128 lanes that this warp may read
    const int row = q * 32 + lane;
    // a tile may cover fewer rows of W than the MMA has (the host spreads a product's rows evenly over the SMs):
    // the accumulator's other rows hold what the stage's unwritten rows happened to contain and are never stored
    const int feature = MODE == 1 ? tile_f * p.tile_rows + (row & 63) : tile_f * p.tile_rows + row;
    const bool feature_ok = (MODE == 1 ? (row & 63) : row) < p.tile_rows && feature < p.n_out;
    float* stage = reinterpret_cast<float*>(smem);  // [BN][BM] partial sums for the cluster reduction (stages are idle by then)
    if (splits > 1 && SCATTER) cluster_wait();
    const unsigned my_rank = splits > 1 ? cluster_rank() : 0;
    const int owned = p.tile_rows / splits;    // SCATTER: rows of the tile that each CTA of the cluster sums and stores
    const unsigned owner = (unsigned)(row / owned);   // per lane: with eight CTAs a warp's rows have two owners
    const int row_local = row - (int)owner * owned;
    if constexpr (MODE == 1) {
        // Gated form (one CTA per tile, no cluster): lanes 0..63 of the accumulator hold 64 features of the
        // gate product, lanes 64..127 the same features of the up product.  The upper two warps hand their
        // values over through shared memory; the lower two compute silu(gate) * up and store.  Both factors
        // are rounded to bfloat16 first, as they are when the product and the gate run as two kernels.
        if (warp >= 2) {
            asm volatile("griddepcontrol.wait;" ::: "memory");   // y may still be read by the predecessor
            // the row scales of scaled rows: their parts are added up in a fixed order while the weights stream in
            if constexpr (BN <= 32) {
                const int e = (int)threadIdx.x - 64;   // 0..127 over the four read-back warps
                if (p.in_ssq != nullptr) {
                    const int tok = e & 31, grp = e >> 5;
                    float acc = 0.0f;
#pragma unroll 8
                    for (int part = grp; part < p.n_in_parts; part += 4) acc += p.in_ssq[(long)part * SSQ_LD + tok];
                    fold[grp * SSQ_LD + tok] = acc;
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (e < 32)
                        fold[8 * SSQ_LD + e] = 1.0f / sqrtf((((fold[e] + fold[SSQ_LD + e]) + fold[2 * SSQ_LD + e]) +
                                                              fold[3 * SSQ_LD + e]) * p.in_inv_width + p.in_eps);
                } else if (e < 32) {
                    fold[8 * SSQ_LD + e] = 1.0f;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
            const float* inv_s = fold + 8 * SSQ_LD;
            ok = nkb > 0 ? mbar_wait(accum, 0, 3) : true;
            ok = __all_sync(0xffffffffu, ok);   // one answer per warp: the tensor-memory loads below are warp-wide
            fence_after();
            float* up_vals = recv;              // [BN][64]
            if (ok && q >= 2) {
#pragma unroll 1
                for (int c0 = 0; c0 < BN && tile_t * BN + c0 < p.n_tok; c0 += 16) {
                    float v[16];
                    if (nkb > 0) tmem_ld16(tmem + ((unsigned)(q * 32) << 16) + c0, v);
                    else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = 0.0f;
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) up_vals[(c0 + j) * 64 + (row - 64)] = v[j];
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");   // the four epilogue warps
            if (ok && q < 2) {                  // whole warps: the tensor-memory load below is warp-wide
                const bool store = feature_ok && g_error == 0;
#pragma unroll 1
                for (int c0 = 0; c0 < BN && tile_t * BN + c0 < p.n_tok; c0 += 16) {
                    float v[16];
                    if (nkb > 0) tmem_ld16(tmem + ((unsigned)(q * 32) << 16) + c0, v);
                    else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = 0.0f;
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int tok = tile_t * BN + c0 + j;
                        if (tok < p.n_tok && store) {
                            const float inv = BN <= 32 ? inv_s[c0 + j] : 1.0f;
                            const float g = __bfloat162float(__float2bfloat16_rn(v[j] * inv));
                            const float u = __bfloat162float(__float2bfloat16_rn(up_vals[(c0 + j) * 64 + row] * inv));
                            reinterpret_cast<__nv_bfloat16*>(p.y)[(long)tok * p.ldy + feature] =
                                __float2bfloat16_rn(g / (1.0f + expf(-g)) * u);
                        }
                    }
                }
            }
        }
    } else {
    constexpr int KEEP = BN <= 32 ? BN : 1;        // a sink's old values that a thread keeps (the folded forms only)
    constexpr int UNROLL = BN <= 32 ? 2 : 1;      // their loops over the tokens are unrolled, so that these stay registers
    float old_s[KEEP], w_sink = 0.0f;
#pragma unroll
    for (int j = 0; j < KEEP; ++j) old_s[j] = 0.0f;
    if (warp >= 2) {
        asm volatile("griddepcontrol.wait;" ::: "memory");   // y may still be read by the predecessor
        // the row scales of scaled rows: their parts are added up in a fixed order while the weights stream in
        if constexpr (BN <= 32) {
            const int e = (int)threadIdx.x - 64;   // 0..127 over the four read-back warps
            if (p.in_ssq != nullptr) {
                const int tok = e & 31, grp = e >> 5;
                float acc = 0.0f;
#pragma unroll 8
                for (int part = grp; part < p.n_in_parts; part += 4) acc += p.in_ssq[(long)part * SSQ_LD + tok];
                fold[grp * SSQ_LD + tok] = acc;
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (e < 32)
                    fold[8 * SSQ_LD + e] = 1.0f / sqrtf((((fold[e] + fold[SSQ_LD + e]) + fold[2 * SSQ_LD + e]) +
                                                          fold[3 * SSQ_LD + e]) * p.in_inv_width + p.in_eps);
            } else if (e < 32) {
                fold[8 * SSQ_LD + e] = 1.0f;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        // a sink's stream and weight, for the values that this thread will finish, fetched while the weights stream in
        if constexpr (BN <= 32) {
            if (p.residual != nullptr && feature_ok && (splits == 1 || owner == my_rank)) {
                w_sink = sink_weight(p, feature);
#pragma unroll
                for (int j = 0; j < KEEP; ++j)
                    if (tile_t * BN + j < p.n_tok) old_s[j] = p.residual[(long)(tile_t * BN + j) * p.ld_res + feature];
            }
        }
        ok = nkb > 0 ? mbar_wait(accum, 0, 3) : true;
        ok = __all_sync(0xffffffffu, ok);       // one answer per warp: the tensor-memory loads below are warp-wide
        fence_after();
        if (ok) {
#pragma unroll UNROLL
            for (int c0 = 0; c0 < BN; c0 += 16) {
                float v[16];
                if (nkb > 0) tmem_ld16(tmem + ((unsigned)(q * 32) << 16) + c0, v);
                else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = 0.0f;
                }
                if (splits > 1 && SCATTER) {
                    // this warp's 32 rows go to the CTA that owns them (which may be this one)
                    if (tile_t * BN + c0 < p.n_tok && row < p.tile_rows) {
                        float* slot = recv + ((size_t)my_rank * BN + c0) * owned + row_local;
                        if (owner == my_rank) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) slot[j * owned] = v[j];
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (tile_t * BN + c0 + j < p.n_tok) st_remote_f32(smem_u32(slot + j * owned), owner, v[j]);
                        }
                    }
                } else if (splits > 1) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) stage[(c0 + j) * BM + row] = v[j];
                } else {
                    float ssq[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int tok = tile_t * BN + c0 + j;
                        ssq[j] = 0.0f;
                        if (tok < p.n_tok && feature_ok) {
                            const float o = BN <= 32 ? finish_value(p, v[j], tok, feature, fold[8 * SSQ_LD + c0 + j],
                                                                    old_s[(c0 + j) % KEEP], w_sink, ssq[j]) : v[j];
                            if (p.y_is_f32) reinterpret_cast<float*>(p.y)[(long)tok * p.ldy + feature] = o;
                            else reinterpret_cast<__nv_bfloat16*>(p.y)[(long)tok * p.ldy + feature] = __float2bfloat16_rn(o);
                        }
                    }
                    if (BN <= 32 && p.residual != nullptr) {   // this warp's part of the rows' sums of squares
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float t = ib_warp_sum(ssq[j]);
                            if (lane == 0) fold[q * SSQ_LD + c0 + j] = t;
                        }
                    }
                }
            }
        }
    }
    // the sink's list of parts: one part per CTA, the four warps' shares added in a fixed order
    auto store_ssq_part = [&]() {
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int e = (int)threadIdx.x - 64;
        if (e < SSQ_LD) {
            const float t = e < BN ? ((fold[e] + fold[SSQ_LD + e]) + fold[2 * SSQ_LD + e]) + fold[3 * SSQ_LD + e] : 0.0f;
            p.out_ssq[((long)tile_f * splits + my_rank) * SSQ_LD + e] = t;
        }
    };
    if constexpr (BN <= 32) {
        if (splits == 1 && p.residual != nullptr && warp >= 2) store_ssq_part();
    }
    if (splits > 1 && SCATTER) {
        cluster_sync_all();                    // every part of the rows this CTA owns is in its shared memory
        if (warp >= 2) {
            const bool mine = owner == my_rank && feature_ok && g_error == 0;
#pragma unroll UNROLL
            for (int c0 = 0; c0 < BN; c0 += 16) {
                if (tile_t * BN + c0 >= p.n_tok) break;
                float sum[16], ssq[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) sum[j] = ssq[j] = 0.0f;
                if (mine) {
                    for (int r = 0; r < splits; ++r) {   // in the order of the ranks, whoever does the adding
                        const float* part = recv + ((size_t)r * BN + c0) * owned + row_local;
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (tile_t * BN + c0 + j < p.n_tok) sum[j] += part[j * owned];
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int tok = tile_t * BN + c0 + j;
                        if (tok < p.n_tok) {
                            const float o = finish_value(p, sum[j], tok, feature, fold[8 * SSQ_LD + c0 + j],
                                                         old_s[(c0 + j) % KEEP], w_sink, ssq[j]);
                            if (p.y_is_f32) reinterpret_cast<float*>(p.y)[(long)tok * p.ldy + feature] = o;
                            else reinterpret_cast<__nv_bfloat16*>(p.y)[(long)tok * p.ldy + feature] = __float2bfloat16_rn(o);
                        }
                    }
                }
                if (p.residual != nullptr) {   // this warp's part of the rows' sums of squares (its own rows only)
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float t = ib_warp_sum(ssq[j]);
                        if (lane == 0) fold[q * SSQ_LD + c0 + j] = t;
                    }
                }
            }
            if (p.residual != nullptr) store_ssq_part();
        }
        // nobody touches another CTA's shared memory after the barrier: the CTAs may leave in any order
    } else if (splits > 1) {
        cluster_sync_all();                    // every CTA's partial sums are in its shared memory
        if (warp >= 2 && my_rank == 0 && feature_ok && g_error == 0) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN && tile_t * BN + c0 < p.n_tok; c0 += 16) {
                float sum[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) sum[j] = stage[(c0 + j) * BM + row];
                for (int r = 1; r < splits; ++r) {   // sixteen independent remote loads at a time
                    float part[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) part[j] = ld_remote_f32(smem_u32(&stage[(c0 + j) * BM + row]), r);
#pragma unroll
                    for (int j = 0; j < 16; ++j) sum[j] += part[j];
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int tok = tile_t * BN + c0 + j;
                    if (tok < p.n_tok) {
                        if (p.y_is_f32) reinterpret_cast<float*>(p.y)[(long)tok * p.ldy + feature] = sum[j];
                        else reinterpret_cast<__nv_bfloat16*>(p.y)[(long)tok * p.ldy + feature] = __float2bfloat16_rn(sum[j]);
                    }
                }
            }
        }
        cluster_sync_all();                    // the first CTA has read its neighbours' shared memory
    }

    }

    if (!ok) {   // a wait of this CTA ran out: copies still in flight get time to land before it leaves
        // a wait ran out somewhere: give copies that are still in flight time to land before the CTA leaves
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    fence_before();
    __syncthreads();
    if (warp == 1) {
        fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// a row-major [rows, k] bfloat16 matrix with row stride ld (elements), boxes of [box_rows, 64]
static bool make_map(CUtensorMap* map, const void* base, long rows, long k, long ld, int box_rows) {
    EncodeTiled enc = encode_fn();
    if (enc == nullptr) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, int STAGES>
constexpr size_t smem_bytes() {
    return (size_t)STAGES * (A_BYTES + BN * BK * 2) + (2 * STAGES + 2) * 8 + 1024 + 9 * SSQ_LD * 4 +
           (BN <= 32 ? (size_t)BN * BM * 4 : 0);   // + the folded forms' sums + the parts received from the cluster
}

template <int BN, int STAGES, int MODE>
static int allow_smem() {
    static IbDeviceSet configured;   // the attribute is kept per device
    return ib_allow_dynamic_smem(configured, gemm_kernel<BN, STAGES, MODE>, smem_bytes<BN, STAGES>());
}

// A kernel with this file's block size, two CTAs per SM and no tensor memory; it is never launched.  The driver's
// occupancy query answers "one CTA per SM" for every kernel that allocates tensor memory, although two CTAs of the
// kernels above run on an SM (each takes 32 or 64 of the 512 columns, and a profile of the 192 CTAs of a gated
// product counts 7.7 active warps per SM: two CTAs on 44 SMs, one on the rest).  So the query is put to this kernel
// with the same shared memory instead.
__global__ void __launch_bounds__(THREADS, 2) occupancy_stand_in(float* p) {
    extern __shared__ float stand_in_smem[];
    stand_in_smem[threadIdx.x] = p[threadIdx.x];
    __syncthreads();
    p[threadIdx.x] = stand_in_smem[THREADS - 1 - threadIdx.x];
}

// CTAs with `smem` bytes of shared memory (two fit on an SM) that the GPU holds at a time when they come in clusters
// of `splits`; 0: not known.  With clusters it is fewer than twice the SMs, because a cluster wants its SMs in one
// part of the chip: 284 in clusters of four and 264 in clusters of eight on a B200 with 148 SMs.
static int resident_ctas(size_t smem, int splits) {
    static int cached[64][9] = {};
    int dev = 0;
    if (splits < 1 || splits > 8 || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (cached[dev][splits] == 0) {
        cached[dev][splits] = -1;
        if (cudaFuncSetAttribute(occupancy_stand_in, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(1, 1, splits);
            cfg.blockDim = dim3(THREADS);
            cfg.dynamicSmemBytes = smem;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 1;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = splits;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, occupancy_stand_in, &cfg) == cudaSuccess && clusters > 0)
                cached[dev][splits] = clusters * splits;
        }
        (void)cudaGetLastError();
    }
    return cached[dev][splits] > 0 ? cached[dev][splits] : 0;
}

template <int BN, int STAGES, int MODE = 0>
static int launch(const CUtensorMap& mw, const CUtensorMap& mx, const Params& p, int splits, cudaStream_t stream) {
    constexpr size_t smem = smem_bytes<BN, STAGES>();
    if (const int e = allow_smem<BN, STAGES, MODE>()) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((p.n_out + p.tile_rows - 1) / p.tile_rows, (p.n_tok + BN - 1) / BN, splits);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = splits;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_kernel<BN, STAGES, MODE>, mw, mx, p);
    return e == cudaSuccess ? ib_launch_status() : (int)e;
}

}  // namespace tc

// How many CTAs share one output tile when the caller does not say
static int choose_splits(int n_tok, int n_out, int num_kb, int bn, int split_k) {
    int splits = split_k;
    if (splits <= 0) {
        const long tiles = (long)((n_out + tc::BM - 1) / tc::BM) * ((n_tok + bn - 1) / bn);
        // few tiles over a long K (the down projection of a decode step): eight parts, of which each CTA has a
        // larger share on its way before the kernel before it has finished; over a short K eight cost more
        // in the cluster's summing than they gain
        splits = tiles >= 120 ? 1 : tiles >= 60 ? 2 : (tiles < 40 && num_kb >= 128) ? 8 : 4;
    }
    if (bn == 256) splits = 1;
    while (splits > 1 && (num_kb + splits - 1) / splits * (splits - 1) >= num_kb) splits >>= 1;  // no empty part
    if (splits == 8 && bn > 32) splits = 4;               // eight only where the owners sum the parts
    return splits;
}

static int g_even_tiles = 1;   // host: see ib_gemm_tcgen05_set_even_tiles

static int sm_count() {
    static int sms[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (sms[dev] == 0 && cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms[dev] = 148;
    return sms[dev];
}

// Rows of W per tile.  A product whose CTAs all fit on the GPU at once, but are more than the SMs, streams its weights
// unevenly: 192 tiles leave 44 SMs with two CTAs and 104 with one, and the product ends when the 44 do.  The tiles
// of such a product are made lower than the MMA (which then computes rows that nobody stores) until there are as
// many CTAs as the GPU holds.  `full` is the MMA's share of rows per tile: 128, or 64 of each matrix in the gated
// form; `resident` what resident_ctas() says for the kernel that will run.
static int tile_rows_for(int n_out, int splits, int full, int resident) {
    if (!g_even_tiles || resident <= 0) return full;
    const long ctas_full = (long)((n_out + full - 1) / full) * splits;
    if (ctas_full > resident || ctas_full <= sm_count()) return full;   // several waves anyway, or one CTA per SM at most   // several waves anyway, or one CTA per SM at most
    const int tiles_wanted = resident / splits;
    int rows = (n_out + tiles_wanted - 1) / tiles_wanted;
    rows = (rows + 7) / 8 * 8;                              // a few CTAs fewer than fit: the next kernel's first ones find room
    rows = (rows + splits - 1) / splits * splits;           // the owners of a cluster take equal shares
    return rows < full ? rows : full;
}

// what resident_ctas() says for the kernel that a product of bn tokens per tile runs (up to 64 tokens: beyond, a
// product has one CTA per SM and tiles as high as the MMA).  The three kernels' shared memory differs by a few KB and
// two of each fit on an SM, so the largest stands for all.
static int resident_for(int bn, int splits) {
    return bn <= 64 ? tc::resident_ctas(tc::smem_bytes<16, 5>(), splits) : 0;
}

static int bn_for(int n_tok) { return n_tok <= 16 ? 16 : n_tok <= 32 ? 32 : n_tok <= 64 ? 64 : n_tok <= 128 ? 128 : 256; }

// The folded forms (see the head of this file) as the exported functions take them: both optional.
struct Folded {
    const float* in_ssq; int n_in_parts; float in_eps; int in_width;          // scaled rows
    float* residual; long ld_res; const void* sink_w; int sink_w_is_f32; float* out_ssq;   // sink
};

static int gemm_tn(const void* x, long ldx, const void* w, long ldw, void* y, long ldy, int y_is_f32, int n_tok,
                   int n_out, int k, int split_k, const Folded& f, cudaStream_t stream) {
    if (n_tok <= 0 || n_out <= 0) return IB_OK;
    if (k <= 0) return IB_ERR_ARGUMENT;
    // TMA wants 16-byte aligned bases and row strides
    if ((k % 8) || (ldx % 8) || (ldw % 8) || ((uintptr_t)x % 16) || ((uintptr_t)w % 16)) return IB_ERR_UNSUPPORTED;
    const int bn = bn_for(n_tok);
    if ((f.in_ssq != nullptr || f.residual != nullptr) && bn > 32) return IB_ERR_UNSUPPORTED;
    if (f.residual != nullptr && (f.sink_w == nullptr || f.out_ssq == nullptr || y_is_f32)) return IB_ERR_ARGUMENT;
    if (f.in_ssq != nullptr && (f.n_in_parts <= 0 || f.in_width <= 0)) return IB_ERR_ARGUMENT;
    tc::Params p;
    p.y = y; p.ldy = ldy; p.n_tok = n_tok; p.n_out = n_out; p.num_kb = (k + tc::BK - 1) / tc::BK; p.y_is_f32 = y_is_f32;
    p.inner = 0;
    p.in_ssq = f.in_ssq; p.n_in_parts = f.n_in_parts; p.in_eps = f.in_eps; p.in_inv_width = f.in_width > 0 ? 1.0f / (float)f.in_width : 0.0f;
    p.residual = f.residual; p.ld_res = f.ld_res; p.sink_w = f.sink_w; p.sink_w_is_f32 = f.sink_w_is_f32; p.out_ssq = f.out_ssq;
    const int splits = choose_splits(n_tok, n_out, p.num_kb, bn, split_k);
    if (splits != 1 && splits != 2 && splits != 4 && splits != 8) return IB_ERR_ARGUMENT;
    p.tile_rows = tile_rows_for(n_out, splits, tc::BM, resident_for(bn, splits));
    CUtensorMap mw, mx;
    if (!tc::make_map(&mw, w, n_out, k, ldw, p.tile_rows) || !tc::make_map(&mx, x, n_tok, k, ldx, bn)) return IB_ERR_UNSUPPORTED;
    switch (bn) {
        // up to 64 tokens: two CTAs per SM with half the ring each, so that tile counts between one and two
        // per SM still run as one wave in which every CTA gets the same share of the memory bandwidth
        case 16: return tc::launch<16, 5>(mw, mx, p, splits, stream);
        case 32: return tc::launch<32, 4>(mw, mx, p, splits, stream);
        case 64: return tc::launch<64, 4>(mw, mx, p, splits, stream);
        case 128: return tc::launch<128, 6>(mw, mx, p, splits, stream);
        default: return tc::launch<256, 4>(mw, mx, p, splits, stream);
    }
}

// x [n_tok, k] (row stride ldx), w [n_out, k] (row stride ldw), both bfloat16; y [n_tok, n_out] bfloat16 or float32.
// split_k: 0 lets the function choose (1, 2, 4 or 8 CTAs per output tile); 8 is taken for up to 32 tokens (4 stands in beyond).
IB_EXPORT int ib_gemm_tn_tcgen05(const void* x, long ldx, const void* w, long ldw, void* y, long ldy, int y_is_f32,
                                 int n_tok, int n_out, int k, int split_k, cudaStream_t stream) {
    const Folded none = {nullptr, 0, 0.0f, 0, nullptr, 0, nullptr, 0, nullptr};
    return gemm_tn(x, ldx, w, ldw, y, ldy, y_is_f32, n_tok, n_out, k, split_k, none, stream);
}

// The same with the norms around it folded in (up to 32 tokens; y bfloat16).  in_ssq (or null): x holds rows times a
// norm's weight, and the n_in_parts parts [.., 32] of their sums of squares over in_width elements; the product is
// scaled by 1 / sqrt(sum / in_width + in_eps) per token.  residual (or null): y is added to this float32 stream
// [n_tok, n_out] (row stride ld_res) in place, what is stored at y is the stream times sink_w [n_out], and the parts
// of the new rows' sums of squares go to out_ssq [ib_gemm_tcgen05_ssq_parts(...), 32].
IB_EXPORT int ib_gemm_tn_tcgen05_folded(const void* x, long ldx, const void* w, long ldw, void* y, long ldy, int n_tok,
                                        int n_out, int k, int split_k, const float* in_ssq, int n_in_parts, float in_eps,
                                        int in_width, float* residual, long ld_res, const void* sink_w,
                                        int sink_w_is_f32, float* out_ssq, cudaStream_t stream) {
    const Folded f = {in_ssq, n_in_parts, in_eps, in_width, residual, ld_res, sink_w, sink_w_is_f32, out_ssq};
    return gemm_tn(x, ldx, w, ldw, y, ldy, 0, n_tok, n_out, k, split_k, f, stream);
}

// Parts that a sink of these sizes writes (one per CTA of the product); negative: the sizes take no sink.
IB_EXPORT int ib_gemm_tcgen05_ssq_parts(int n_tok, int n_out, int k, int split_k) {
    if (n_tok <= 0 || n_out <= 0 || k <= 0) return IB_ERR_ARGUMENT;
    const int bn = bn_for(n_tok);
    if (bn > 32) return IB_ERR_UNSUPPORTED;
    const int splits = choose_splits(n_tok, n_out, (k + tc::BK - 1) / tc::BK, bn, split_k);
    const int rows = tile_rows_for(n_out, splits, tc::BM, resident_for(bn, splits));
    return ((n_out + rows - 1) / rows) * splits;
}

// y[t, f] = silu(x[t] . w[f]) * (x[t] . w[inner + f]) for f < inner: the gate and up products of a gated feed-forward
// and the gate itself in one kernel.  w [2 * inner, k] holds the gate matrix above the up matrix; y [n_tok, inner]
// bfloat16.  Up to 32 tokens (IB_ERR_UNSUPPORTED beyond; the caller then runs product and gate separately).  With
// in_ssq, x holds scaled rows as above and both products are scaled per token before the gate.
IB_EXPORT int ib_gemm_swiglu_tcgen05_folded(const void* x, long ldx, const void* w, long ldw, void* y, long ldy, int n_tok,
                                            int inner, int k, const float* in_ssq, int n_in_parts, float in_eps,
                                            int in_width, cudaStream_t stream) {
    if (n_tok <= 0 || inner <= 0) return IB_OK;
    if (k <= 0) return IB_ERR_ARGUMENT;
    if ((k % 8) || (ldx % 8) || (ldw % 8) || ((uintptr_t)x % 16) || ((uintptr_t)w % 16) || n_tok > 32) return IB_ERR_UNSUPPORTED;
    if (in_ssq != nullptr && (n_in_parts <= 0 || in_width <= 0)) return IB_ERR_ARGUMENT;
    const int bn = n_tok <= 16 ? 16 : 32;
    tc::Params p;
    p.y = y; p.ldy = ldy; p.n_tok = n_tok; p.n_out = inner; p.num_kb = (k + tc::BK - 1) / tc::BK; p.y_is_f32 = 0;
    p.inner = inner;
    p.in_ssq = in_ssq; p.n_in_parts = n_in_parts; p.in_eps = in_eps; p.in_inv_width = in_width > 0 ? 1.0f / (float)in_width : 0.0f;
    p.residual = nullptr; p.ld_res = 0; p.sink_w = nullptr; p.sink_w_is_f32 = 0; p.out_ssq = nullptr;
    p.tile_rows = tile_rows_for(inner, 1, 64, resident_for(bn, 1));
    CUtensorMap mw, mx;
    if (!tc::make_map(&mw, w, 2L * inner, k, ldw, p.tile_rows) || !tc::make_map(&mx, x, n_tok, k, ldx, bn)) return IB_ERR_UNSUPPORTED;
    return bn == 16 ? tc::launch<16, 5, 1>(mw, mx, p, 1, stream) : tc::launch<32, 4, 1>(mw, mx, p, 1, stream);
}

IB_EXPORT int ib_gemm_swiglu_tcgen05(const void* x, long ldx, const void* w, long ldw, void* y, long ldy, int n_tok,
                                     int inner, int k, cudaStream_t stream) {
    return ib_gemm_swiglu_tcgen05_folded(x, ldx, w, ldw, y, ldy, n_tok, inner, k, nullptr, 0, 0.0f, 0, stream);
}

// 1: later launches may start before the kernel before them in the stream has finished (programmatic dependent
// launch); they read their weights at once and wait for that kernel before they touch anything else.  Every
// kernel that runs between two such launches must itself call griddepcontrol.wait before its first access to
// memory that another kernel writes.  0 (default): plain stream order.
IB_EXPORT void ib_gemm_tcgen05_set_pdl(int on) { tc::g_pdl = on; }

// 1 (default): a product whose CTAs all run at once gets tiles of such a height that every SM has the same number
// of them; 0: every tile is as high as the MMA.  The number of parts that a sink writes follows the setting, so it
// is set before the lists of parts are sized.
IB_EXPORT void ib_gemm_tcgen05_set_even_tiles(int on) { g_even_tiles = on; }

// What the choice of a product's tiles rests on: the CTAs that the GPU holds at a time of the kernel that a product of
// n_tok tokens runs (gated: the gate/up form), in clusters of `splits`; and the rows of W per tile that follow.
IB_EXPORT int ib_gemm_tcgen05_resident_ctas(int n_tok, int gated, int splits) {
    return resident_for(gated ? (n_tok <= 16 ? 16 : 32) : bn_for(n_tok), splits);
}
IB_EXPORT int ib_gemm_tcgen05_tile_rows(int n_tok, int n_out, int k, int split_k, int gated) {
    if (n_tok <= 0 || n_out <= 0 || k <= 0) return IB_ERR_ARGUMENT;
    if (gated) return tile_rows_for(n_out, 1, 64, resident_for(n_tok <= 16 ? 16 : 32, 1));
    const int bn = bn_for(n_tok);
    const int splits = choose_splits(n_tok, n_out, (k + tc::BK - 1) / tc::BK, bn, split_k);
    return tile_rows_for(n_out, splits, tc::BM, resident_for(bn, splits));
}

// The error word of the kernels above: 0, or the code of the first wait that ran out (1 producer, 2 MMA
// issuer, 3 epilogue).  Reading it synchronises with the device; `reset` clears it.
IB_EXPORT int ib_gemm_tcgen05_error(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, tc::g_error, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(tc::g_error, &zero, sizeof(int));
    }
    return v;
}

// The same word on its way to `out` (pinned host memory) in stream order, without waiting for the device: the
// caller reads it after an event that it records behind this call.
IB_EXPORT int ib_gemm_tcgen05_error_async(int* out, cudaStream_t stream) {
    return (int)cudaMemcpyFromSymbolAsync(out, tc::g_error, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
}


#endif
