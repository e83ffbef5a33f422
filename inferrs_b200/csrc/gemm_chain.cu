// A chain of matrix products for a few tokens as ONE persistent kernel: y_p[t, f] = sum_k x_p[t, k] * w_p[f, k] for
// p = 0 .. n - 1, where the input of a product is the output of the one before it (or was there before the launch).
//
// A decode step of a handful of tokens is bound by streaming the weights, and a layer's products are too small to hide
// what a kernel loses at its ends (the last tiles' latency, the summing of the parts, the read-back, the first tile of
// activations): 4 to 6 us each against 5 to 30 us of streaming.  Here one CTA per SM stays for the whole chain and its
// weight producer never stops: while the CTAs meet between two products, the next product's weights, which depend on
// nothing, already fill the ring.
//
// Work: the units of a product are its 128x64 blocks of W (with the matching 16x64 block of x), tile after tile,
// k-block after k-block, in one line; CTA c takes the c-th equal slice of every product's line, so every SM reads the
// same number of bytes whatever the shapes.  A slice that does not end its tile yields a partial sum in a float32
// workspace in global memory; the CTA that holds the tile's last k-blocks adds the parts in the order of the CTAs (the
// same inputs give the same bits) and finishes the tile.  The workspace holds a "not yet" value wherever nothing has
// been written, so the parts need no flag and no fence: the finisher reads until no value says "not yet", then writes
// "not yet" back.  Finishing can fold the norms around a product in, as the single-product kernel does
// (gemm_tcgen05.cu): "scaled rows" in (the accumulator is scaled per token by a row scale made from parts of sums of
// squares), a "sink" out (the result is added to the float32 residual stream, and the stream times the next norm's
// weight is stored with the parts of the new sums of squares), or the gate of a gated feed-forward (a tile is 64 rows
// of the gate matrix above the same 64 rows of the up matrix).
//
// Between two products every CTA says at a counter in global memory that it has finished its tiles; the activations'
// producer waits there (the weights go on) before it fetches the next product's activations.  CTAs of one launch wait
// for each other, so the launch is cooperative: all its CTAs are resident.  Per CTA: warp 0 = weights (two lanes, one
// per half tile, in one instruction), warp 1 = MMA issuer (two accumulators in tensor memory in turn), warps 2..5 =
// read-back and finishing, warp 6 = activations.
//
// All waits are bounded (about two seconds): mbarrier waits (codes 1 to 4), the finisher's wait for the parts (5), the
// activations' wait at a counter (6).  A wait that runs out records its code in the library's error word; the CTA then
// lets copies in flight land, frees its tensor memory and returns.
#include <cuda.h>

#include "common.cuh"
#include "sm100.cuh"

#if IB_ACT_BF16

namespace ch {

using namespace sm100;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int BN = 16;          // tokens
constexpr int UMMA_K = 16;
constexpr int THREADS = 224;   // warp 0: weights, 1: products, 2 to 5: read-back, 6: activations
constexpr int STAGES = 10;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BN * BK * 2;
constexpr int MAX_PHASES = 4;
constexpr int SSQ_LD = 32;      // tokens per part of a list of sums of squares, as in gemm_tcgen05.cu
constexpr int SLOT = BN * BM;   // floats of one partial sum: [token][row]

__device__ int g_error = 0;
static int g_pdl = 0;

__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, int code) {
    return mbar_wait_bounded(bar, parity, &g_error, code);
}
__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }  // warps 2..5
__device__ __forceinline__ bool epilogue_all(bool mine) {   // the same barrier, and whether every thread says yes
    unsigned all;
    asm volatile("{\n.reg .pred p, q;\nsetp.ne.u32 p, %1, 0;\nbar.red.and.pred q, 1, 128, p;\nselp.u32 %0, 1, 0, q;\n}"
                 : "=r"(all) : "r"((unsigned)mine) : "memory");
    return all != 0;
}
__device__ __forceinline__ int ld_acquire(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
constexpr unsigned NOT_YET = 0xffc0deadu;   // a NaN that no sum comes out as: "this value has not been written"
// Four values in one access, answered by the L2 cache (where other SMs' stores arrive), never by this SM's own cache.
// (A weak load on purpose: loads marked volatile or relaxed went out one after the other, each waiting for the one before
// it, and a dozen of them took two microseconds.)
__device__ __forceinline__ uint4 ld_l2_quad(const float* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

struct Phase {
    void* y;                  // [n_tok, n_out] bfloat16 (gated: [n_tok, inner])
    long ldy;
    int n_out;                // features stored (gated: inner)
    int num_kb;               // k-blocks of 64
    int tiles;                // output tiles (plain: 128 features each; gated: 64 features each)
    int gated;                // 1: w holds the gate matrix above the up matrix; a tile is 64 + 64 of their rows
    int inner;
    long total_units;         // tiles * num_kb
    // scaled rows in (null: x is used as it is)
    const float* in_ssq;
    int n_in_parts;
    float in_eps, in_inv_width;
    // sink out (null: y is stored as it is)
    float* residual;
    long ld_res;
    const void* sink_w;
    int sink_w_is_f32;
    float* out_ssq;           // [tiles][SSQ_LD]
};

struct Params {
    Phase ph[MAX_PHASES];
    int n_phases, n_tok;
    float* scratch;           // [grid][SLOT], all NOT_YET between launches: per CTA a slice that does not end its tile, [row][token]
    int* bars;                // [MAX_PHASES + 1], zero between launches: CTAs that have finished product p; the last: CTAs that left
};

struct Maps {
    CUtensorMap w[MAX_PHASES], x[MAX_PHASES];
};

__device__ __forceinline__ long slice_begin(long total, int grid, int c) { return total * c / grid; }

__global__ void __launch_bounds__(THREADS, 1) chain_kernel(const __grid_constant__ Maps maps, const Params p) {
    extern __shared__ unsigned char raw_smem[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~(uintptr_t)1023);
    unsigned char* a_tiles = smem;
    unsigned char* b_tiles = smem + STAGES * A_BYTES;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(b_tiles + STAGES * B_BYTES);
    const unsigned full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const unsigned accf0 = smem_u32(bars + 2 * STAGES), acce0 = smem_u32(bars + 2 * STAGES + 2);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * STAGES + 4);
    float* fold = reinterpret_cast<float*>(bars + 2 * STAGES + 5);   // [4][SSQ_LD] partial sums, [SSQ_LD] row scales
    float* own_head = fold + 5 * SSQ_LD;      // this CTA's own slice of the tile it finishes last, [token][row]
    float* own_whole = own_head + SLOT;       // a tile that this CTA computes alone

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cta = blockIdx.x, grid = gridDim.x;

    // the kernel after this one may start its own prologue; this one reads weights at once and everything else
    // only after griddepcontrol.wait
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 2); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(accf0 + 8 * b, 1); mbar_init(acce0 + 8 * b, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(32) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before();
    __syncthreads();
    fence_after();
    const unsigned tmem = *tmem_slot;
    bool ok = true;

    // A thread gets a bulk copy accepted about every 400 cycles, however small the copy is: one thread that asks for the
    // weights and the activations of a stage (three copies) feeds an SM a third of what the memory can give it.  So the
    // two halves of a weight tile are asked for by two lanes in one instruction, and the activations by another warp.
    struct Cursor { int ph, u, e, tile, kb, num_kb, gated, inner; };
    const int n_phases = p.n_phases;
    auto enter = [&](Cursor& c) {                                 // the cursor's slice of product c.ph, or the next that has one
        while (c.ph < n_phases) {
            const Phase& f = p.ph[c.ph];
            c.u = (int)slice_begin(f.total_units, grid, cta);
            c.e = (int)slice_begin(f.total_units, grid, cta + 1);
            if (c.u < c.e) {
                c.num_kb = f.num_kb; c.gated = f.gated; c.inner = f.inner;   // kept in registers: a look into the
                c.tile = c.u / c.num_kb;                                      // parameters with a running index is slow
                c.kb = c.u - c.tile * c.num_kb;
                return;
            }
            ++c.ph;
        }
    };
    auto advance = [&](Cursor& c) {
        if (++c.u >= c.e) {
            ++c.ph;
            enter(c);
        } else if (++c.kb == c.num_kb) {
            c.kb = 0;
            ++c.tile;
        }
    };

    if (warp == 0) {
        if (lane < 2) {
            // weights, as far ahead as the ring allows; they wait for nobody but the ring
            const unsigned pair = 0x3u;
            const unsigned long long pol = policy_evict_first();
            Cursor c{0, 0, 0, 0, 0, 1, 0, 0};
            unsigned s = 0, turn = 0;
            enter(c);
            while (c.ph < n_phases && ok) {
                if (turn > 0) {
                    bool got = true;
                    if (lane == 0) got = mbar_wait(empty0 + 8 * s, (turn - 1) & 1, 1);
                    if (!__shfl_sync(pair, got, 0)) { ok = false; break; }
                }
                if (lane == 0) mbar_expect_tx(full0 + 8 * s, A_BYTES);
                __syncwarp(pair);
                const int row = c.gated ? (lane ? c.inner : 0) + c.tile * 64 : c.tile * BM + lane * 64;
                tma_load_2d_hint(smem_u32(a_tiles + s * A_BYTES) + lane * (A_BYTES / 2), &maps.w[c.ph], c.kb * BK, row,
                                 full0 + 8 * s, pol);
                if (++s == STAGES) { s = 0; ++turn; }
                advance(c);
            }
        }
    } else if (warp == 6) {
        if (lane == 0) {
            // activations: of the first product after the kernels before this one, of the others after every CTA has
            // finished the product before
            Cursor c{0, 0, 0, 0, 0, 1, 0, 0};
            unsigned s = 0, turn = 0;
            int ready = 1;                                        // products 0 .. ready - 1 may fetch activations
            enter(c);
            asm volatile("griddepcontrol.wait;" ::: "memory");
            while (c.ph < n_phases && ok) {
                if (c.ph >= ready) {
                    unsigned long long t0 = 0;
                    for (unsigned it = 1; ld_acquire(p.bars + c.ph - 1) < grid; ++it) {
                        if ((it & 255u) == 0) {
                            const unsigned long long now = global_ns();
                            if (t0 == 0) {
                                t0 = now;
                            } else if (now - t0 > MBAR_WAIT_LIMIT_NS) {
                                atomicCAS(&g_error, 0, 6);
                                ok = false;
                                break;
                            }
                        }
                    }
                    if (!ok) break;
                    ready = c.ph + 1;
                    asm volatile("fence.proxy.async.global;" ::: "memory");   // the copies read what other SMs' threads stored
                }
                if (turn > 0 && !mbar_wait(empty0 + 8 * s, (turn - 1) & 1, 1)) { ok = false; break; }
                mbar_expect_tx(full0 + 8 * s, B_BYTES);
                tma_load_2d(smem_u32(b_tiles + s * B_BYTES), &maps.x[c.ph], c.kb * BK, 0, full0 + 8 * s);
                if (++s == STAGES) { s = 0; ++turn; }
                advance(c);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
            unsigned i = 0, s = 0, turn = 0;
            int seg = 0;
            for (int ph = 0; ph < p.n_phases && ok; ++ph) {
                const Phase& f = p.ph[ph];
                const int u0 = (int)slice_begin(f.total_units, grid, cta), u1 = (int)slice_begin(f.total_units, grid, cta + 1);
                const int num_kb = f.num_kb;
                int kb = u0 % num_kb;
                bool first = true;   // the next MMA starts a slice of a tile
                for (int u = u0; u < u1 && ok; ++u, ++i) {
                    const int buf = seg & 1;
                    if (first && seg >= 2 && !mbar_wait(acce0 + 8 * buf, (unsigned)((seg >> 1) - 1) & 1, 4)) { ok = false; break; }
                    if (!mbar_wait(full0 + 8 * s, turn & 1, 2)) { ok = false; break; }
                    fence_after();
                    const unsigned long long da = desc_k_major(smem_u32(a_tiles + s * A_BYTES));
                    const unsigned long long db = desc_k_major(smem_u32(b_tiles + s * B_BYTES));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma(tmem + buf * BN, da + (unsigned long long)(k * UMMA_K * 2 / 16),
                             db + (unsigned long long)(k * UMMA_K * 2 / 16), idesc, (first && k == 0) ? 0u : 1u);
                    first = false;
                    umma_commit(empty0 + 8 * s);
                    if (++s == STAGES) { s = 0; ++turn; }
                    if (++kb == num_kb || u == u1 - 1) {   // the slice of this tile ends here
                        kb = 0;
                        umma_commit(accf0 + 8 * buf);
                        ++seg;
                        first = true;
                    }
                }
            }
        }
    } else {
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const int e = (int)threadIdx.x - 64;       // 0 .. 127 over the four read-back warps
        const bool leader = e == 0;
        const int n_tok = p.n_tok;
        // A slice that does not end its tile goes to this CTA's slot in global memory, [row][token].  The slot holds
        // NOT_YET wherever nothing has been written: the CTA that finishes the tile reads it until no value is NOT_YET
        // any more, then writes NOT_YET back.  No flag, and no fence between the values and a flag: such a fence took
        // about two microseconds here while the copies of the next product's weights fill the memory system, and it
        // stood at the end of every product.  (A value is four bytes, written at once; sixteen bytes go in one access
        // only to make the accesses few.)
        float* tail = p.scratch + (long)cta * SLOT;
        float* inv_s = fold + 4 * SSQ_LD;
        int seg = 0;
        for (int ph = 0; ph < p.n_phases && ok; ++ph) {
            const Phase f = p.ph[ph];   // a copy in registers
            const int u0 = (int)slice_begin(f.total_units, grid, cta), u1 = (int)slice_begin(f.total_units, grid, cta + 1);
            bool scales_made = false;

            // Finish a tile: add the parts (the slices of the CTAs first_c .. cta - 1 in that order, then this CTA's own
            // part from shared memory), apply what the product folds in, store.  All four warps come here together.
            // What does not depend on the other CTAs (the stream's old values, the norm's weight) is asked for first,
            // and the parts of up to four CTAs are asked for at a time: every question to the L2 cache that waits for the
            // one before it is another half microsecond at the end of a product.
            auto finish_tile = [&](int tile, int first_c, const float* own) {
                const int rows = f.gated ? 64 : BM;
                const int feature = f.gated ? tile * 64 + row : tile * BM + row;
                const bool reads = row < rows;                    // (every row of the slots is read, so that every mark is wiped)
                const bool mine = reads && feature < f.n_out;
                float v[BN], up[BN], ssq[BN], old[BN];
                float w_sink = 0.0f;
#pragma unroll
                for (int j = 0; j < BN; ++j) v[j] = up[j] = ssq[j] = old[j] = 0.0f;
                if (mine && f.residual != nullptr) {
                    w_sink = f.sink_w_is_f32 ? reinterpret_cast<const float*>(f.sink_w)[feature]
                                             : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(f.sink_w)[feature]);
#pragma unroll
                    for (int j = 0; j < BN; ++j)
                        if (j < n_tok) old[j] = __ldcg(f.residual + (long)j * f.ld_res + feature);   // last written by another SM
                }
                if (reads) {
                    constexpr int GROUP = 6, HALF = BN / 2;   // (a tile of these shapes is shared by five or six CTAs)
                    unsigned long long t0 = 0;
                    for (int c = first_c; c < cta && ok; c += GROUP) {
                        const int n_here = cta - c < GROUP ? cta - c : GROUP;
#pragma unroll
                        for (int jh = 0; jh < BN; jh += HALF) {       // eight tokens at a time: the values stay in registers
                            if (jh >= n_tok || !ok) break;
                            uint4 a[GROUP][HALF / 4], b[GROUP][HALF / 4];
                            for (unsigned it = 1;; ++it) {
                                bool all = true;
#pragma unroll
                                for (int g = 0; g < GROUP; ++g) {
                                    if (g < n_here) {
                                        const float* theirs = p.scratch + (long)(c + g) * SLOT + row * BN + jh;
#pragma unroll
                                        for (int j4 = 0; j4 < HALF / 4; ++j4) {
                                            if (jh + j4 * 4 < n_tok) {
                                                a[g][j4] = ld_l2_quad(theirs + j4 * 4);
                                                if (f.gated) b[g][j4] = ld_l2_quad(theirs + 64 * BN + j4 * 4);
                                            }
                                        }
                                    }
                                }
#pragma unroll
                                for (int g = 0; g < GROUP; ++g) {
                                    if (g < n_here) {
#pragma unroll
                                        for (int j4 = 0; j4 < HALF / 4; ++j4) {
                                            const int j = jh + j4 * 4;
                                            if (j < n_tok) {
                                                const uint4 x = a[g][j4];
                                                all = all && x.x != NOT_YET && (j + 1 >= n_tok || x.y != NOT_YET) &&
                                                      (j + 2 >= n_tok || x.z != NOT_YET) && (j + 3 >= n_tok || x.w != NOT_YET);
                                                if (f.gated) {
                                                    const uint4 y = b[g][j4];
                                                    all = all && y.x != NOT_YET && (j + 1 >= n_tok || y.y != NOT_YET) &&
                                                          (j + 2 >= n_tok || y.z != NOT_YET) && (j + 3 >= n_tok || y.w != NOT_YET);
                                                }
                                            }
                                        }
                                    }
                                }
                                if (all) {
                                    break;
                                }
                                __nanosleep(100);
                                if ((it & 255u) == 0) {
                                    const unsigned long long now = global_ns();
                                    if (t0 == 0) {
                                        t0 = now;
                                    } else if (now - t0 > MBAR_WAIT_LIMIT_NS) {
                                        atomicCAS(&g_error, 0, 5);
                                        ok = false;
                                        break;
                                    }
                                }
                            }
                            const uint4 blank = make_uint4(NOT_YET, NOT_YET, NOT_YET, NOT_YET);
#pragma unroll
                            for (int g = 0; g < GROUP; ++g) {
                                if (g < n_here) {
                                    float* theirs = p.scratch + (long)(c + g) * SLOT + row * BN + jh;
#pragma unroll
                                    for (int j4 = 0; j4 < HALF / 4; ++j4) {
                                        const int j = jh + j4 * 4;
                                        if (j < n_tok) {
                                            v[j] += __uint_as_float(a[g][j4].x); v[j + 1] += __uint_as_float(a[g][j4].y);
                                            v[j + 2] += __uint_as_float(a[g][j4].z); v[j + 3] += __uint_as_float(a[g][j4].w);
                                            *reinterpret_cast<uint4*>(theirs + j4 * 4) = blank;
                                            if (f.gated) {
                                                up[j] += __uint_as_float(b[g][j4].x); up[j + 1] += __uint_as_float(b[g][j4].y);
                                                up[j + 2] += __uint_as_float(b[g][j4].z); up[j + 3] += __uint_as_float(b[g][j4].w);
                                                *reinterpret_cast<uint4*>(theirs + 64 * BN + j4 * 4) = blank;
                                            }
                                        }
                                    }
                                }
                            }
                        }
                    }
                }
                ok = epilogue_all(ok);   // (a thread that gave up takes the others with it)
                if (mine && ok) {
#pragma unroll
                    for (int j = 0; j < BN; ++j) {
                        if (j >= n_tok) break;
                        const float inv = inv_s[j];
                        float o = (v[j] + own[j * BM + row]) * inv;
                        if (f.gated) {
                            const float g = __bfloat162float(__float2bfloat16_rn(o));
                            const float u = __bfloat162float(__float2bfloat16_rn((up[j] + own[j * BM + row + 64]) * inv));
                            o = g / (1.0f + expf(-g)) * u;
                        } else if (f.residual != nullptr) {
                            const float s = old[j] + __bfloat162float(__float2bfloat16_rn(o));
                            f.residual[(long)j * f.ld_res + feature] = s;
                            ssq[j] = s * s;
                            o = s * w_sink;
                        }
                        reinterpret_cast<__nv_bfloat16*>(f.y)[(long)j * f.ldy + feature] = __float2bfloat16_rn(o);
                    }
                }
                if (f.residual != nullptr) {   // the tile's part of the rows' sums of squares, the warps' shares in a fixed order
#pragma unroll
                    for (int j = 0; j < BN; ++j) {
                        if (j >= n_tok) break;
                        const float t = ib_warp_sum(ssq[j]);
                        if (lane == 0) fold[q * SSQ_LD + j] = t;
                    }
                    epilogue_sync();
                    if (e < SSQ_LD)
                        f.out_ssq[(long)tile * SSQ_LD + e] =
                            e < n_tok ? ((fold[e] + fold[SSQ_LD + e]) + fold[2 * SSQ_LD + e]) + fold[3 * SSQ_LD + e] : 0.0f;
                    epilogue_sync();
                }
            };

            // The tile whose last k-blocks are this CTA's first slice is finished last; which CTA holds its first
            // k-blocks is worked out now, while the first products run.
            int head_tile = -1, head_first_c = cta;
            if (u0 < u1 && u0 % f.num_kb != 0) {
                const long tile_begin = (long)(u0 / f.num_kb) * f.num_kb;
                int c0 = (int)(tile_begin * grid / f.total_units);
                while (c0 > 0 && slice_begin(f.total_units, grid, c0) > tile_begin) --c0;
                while (slice_begin(f.total_units, grid, c0 + 1) <= tile_begin) ++c0;
                head_first_c = c0;
            }
            for (int u = u0; u < u1 && ok; ++seg) {
                const int tile = u / f.num_kb;
                const int kb_begin = u - tile * f.num_kb;
                const int tile_end = (tile + 1) * f.num_kb;
                const int seg_end = tile_end < u1 ? tile_end : u1;
                const bool ends_tile = seg_end == tile_end;
                const int buf = seg & 1;
                {   // one lane asks, and rests between its questions: 128 threads asking in a loop hold up the
                    // producers' and the MMA thread's own barrier operations
                    bool got = true;
                    if (lane == 0) {
                        const unsigned par = (unsigned)(seg >> 1) & 1;
                        unsigned long long t0 = 0;
                        for (unsigned it = 1; !mbar_test_wait(accf0 + 8 * buf, par); ++it) {
                            __nanosleep(100);
                            if ((it & 1023u) == 0) {
                                const unsigned long long now = global_ns();
                                if (t0 == 0) {
                                    t0 = now;
                                } else if (now - t0 > MBAR_WAIT_LIMIT_NS) {
                                    atomicCAS(&g_error, 0, 3);
                                    got = false;
                                    break;
                                }
                            }
                        }
                    }
                    // (all four warps leave together when one of them has given up: those that stay would wait for it)
                    if (!epilogue_all(__shfl_sync(0xffffffffu, got, 0))) { ok = false; break; }
                }
                fence_after();
                if (!scales_made) {
                    // This product's activations have arrived, so the product before it is finished everywhere: the
                    // parts of its rows' sums of squares are there.  Four groups of threads add them up in a fixed order.
                    scales_made = true;
                    if (f.in_ssq != nullptr) {
                        const int tok = e & 31, grp = e >> 5;
                        float acc = 0.0f;
#pragma unroll 8
                        for (int part = grp; part < f.n_in_parts; part += 4) acc += __ldcg(f.in_ssq + (long)part * SSQ_LD + tok);
                        fold[grp * SSQ_LD + tok] = acc;
                        epilogue_sync();
                        if (e < SSQ_LD)
                            inv_s[e] = 1.0f / sqrtf((((fold[e] + fold[SSQ_LD + e]) + fold[2 * SSQ_LD + e]) + fold[3 * SSQ_LD + e]) *
                                                    f.in_inv_width + f.in_eps);
                    } else if (e < SSQ_LD) {
                        inv_s[e] = 1.0f;
                    }
                    epilogue_sync();
                }
                float v[BN];
                tmem_ld16(tmem + ((unsigned)(q * 32) << 16) + buf * BN, v);
                if (!ends_tile) {
#pragma unroll
                    for (int j = 0; j < BN; j += 4)
                        if (j < n_tok)   // (whole groups of four: the tokens beyond n_tok are zero and nobody reads them)
                            *reinterpret_cast<float4*>(tail + row * BN + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                } else {
                    float* keep = kb_begin > 0 ? own_head : own_whole;
                    if (kb_begin > 0) head_tile = tile;
#pragma unroll
                    for (int j = 0; j < BN; ++j)
                        if (j < n_tok) keep[j * BM + row] = v[j];
                }
                fence_before();
                if (lane == 0) mbar_arrive(acce0 + 8 * buf);   // this warp has read the accumulator
                if (ends_tile && kb_begin == 0) {
                    epilogue_sync();                            // the four warps' shares of the tile are in shared memory
                    finish_tile(tile, cta, own_whole);
                    epilogue_sync();                            // before the next whole tile overwrites them
                }
                u = seg_end;
            }
            // Finish the tile whose last k-blocks were this CTA's first slice.  This comes last, so that no CTA's stream
            // of W waits for another CTA: the parts it needs are written when their CTAs are done streaming.
            if (head_tile >= 0 && ok) {
                epilogue_sync();                                // the four warps' shares of the own part are written
                finish_tile(head_tile, head_first_c, own_head);
            }
            // this CTA has finished its tiles of the product: say so (nobody waits behind the last product)
            if (ph + 1 < p.n_phases && ok) {
                epilogue_sync();
                if (leader) {
                    __threadfence();   // the one fence for what the four warps have stored (the barrier orders it after them)
                    const int old = atomicAdd(p.bars + ph, 1);
                    // the last to arrive knows that everybody has passed the counter before this one: zero it again
                    if (old == grid - 1 && ph > 0) p.bars[ph - 1] = 0;
                }
            }
        }
        // the last CTA to leave zeroes the last counter that was used
        if (leader && p.n_phases > 1) {
            const int old = atomicAdd(p.bars + MAX_PHASES, 1);
            if (old == grid - 1) {
                p.bars[p.n_phases - 2] = 0;
                p.bars[MAX_PHASES] = 0;
            }
        }
    }

    if (!ok) {   // a wait of this CTA ran out: copies still in flight get time to land before it leaves
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    fence_before();
    __syncthreads();
    if (warp == 1) {
        fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(32) : "memory");
    }
}

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

}  // namespace ch

// One product of a chain, as the exported function takes it.
struct IbChainProduct {
    const void* x; long ldx;          // [n_tok, k] bfloat16
    const void* w; long ldw;          // [n_out, k] bfloat16 (gated: [2 * inner, k], the gate matrix above the up matrix)
    void* y; long ldy;                // [n_tok, n_out] bfloat16 (gated: [n_tok, inner])
    int n_out, k, gated;              // gated: n_out is inner
    const float* in_ssq; int n_in_parts; float in_eps; int in_width;                      // scaled rows in, or null
    float* residual; long ld_res; const void* sink_w; int sink_w_is_f32; float* out_ssq;   // sink out, or null
};

// Floats of workspace for `grid` CTAs (plus MAX_PHASES + 1 zeroed ints of counters).
IB_EXPORT long ib_gemm_chain_workspace_floats(int grid) { return (long)grid * ch::SLOT; }
// The 32 bits that every float of the workspace holds between launches.
IB_EXPORT int ib_gemm_chain_workspace_fill() { return (int)ch::NOT_YET; }
IB_EXPORT int ib_gemm_chain_max_products() { return ch::MAX_PHASES; }
// Parts that a sink of a product with n_out features writes: one per tile.
IB_EXPORT int ib_gemm_chain_ssq_parts(int n_out) { return (n_out + ch::BM - 1) / ch::BM; }

// n products (1 .. 4) for n_tok <= 16 tokens as one persistent cooperative kernel of `grid` CTAs (at most one per SM
// and no more than the smallest product has k-blocks).  The workspace and the counters belong to the
// caller; launches that share them must not overlap.  The kernel leaves the workspace filled with its "not yet" value and the counters zero.
IB_EXPORT int ib_gemm_chain(const IbChainProduct* products, int n, int n_tok, float* scratch, int* counters,
                            int grid, cudaStream_t stream) {
    if (n <= 0 || n > ch::MAX_PHASES || n_tok <= 0 || n_tok > ch::BN || grid <= 0) return IB_ERR_UNSUPPORTED;
    if (scratch == nullptr || counters == nullptr) return IB_ERR_ARGUMENT;
    ch::Params p;
    static ch::Maps maps;   // filled per launch; copied into the launch's parameters
    p.n_phases = n; p.n_tok = n_tok; p.scratch = scratch; p.bars = counters;
    for (int i = 0; i < n; ++i) {
        const IbChainProduct& c = products[i];
        if (c.k <= 0 || c.n_out <= 0) return IB_ERR_ARGUMENT;
        if ((c.k % 8) || (c.ldx % 8) || (c.ldw % 8) || ((uintptr_t)c.x % 16) || ((uintptr_t)c.w % 16)) return IB_ERR_UNSUPPORTED;
        if (c.gated && (c.n_out % 64)) return IB_ERR_UNSUPPORTED;
        if (c.residual != nullptr && (c.sink_w == nullptr || c.out_ssq == nullptr || c.gated)) return IB_ERR_ARGUMENT;
        if (c.in_ssq != nullptr && (c.n_in_parts <= 0 || c.in_width <= 0)) return IB_ERR_ARGUMENT;
        ch::Phase& f = p.ph[i];
        f.y = c.y; f.ldy = c.ldy; f.n_out = c.n_out; f.num_kb = (c.k + ch::BK - 1) / ch::BK; f.gated = c.gated;
        f.inner = c.gated ? c.n_out : 0;
        f.tiles = c.gated ? c.n_out / 64 : (c.n_out + ch::BM - 1) / ch::BM;
        f.total_units = (long)f.tiles * f.num_kb;
        if (f.total_units < grid) return IB_ERR_UNSUPPORTED;
        f.in_ssq = c.in_ssq; f.n_in_parts = c.n_in_parts; f.in_eps = c.in_eps;
        f.in_inv_width = c.in_width > 0 ? 1.0f / (float)c.in_width : 0.0f;
        f.residual = c.residual; f.ld_res = c.ld_res; f.sink_w = c.sink_w; f.sink_w_is_f32 = c.sink_w_is_f32; f.out_ssq = c.out_ssq;
        const long w_rows = c.gated ? 2L * c.n_out : c.n_out;
        if (!ch::make_map(&maps.w[i], c.w, w_rows, c.k, c.ldw, 64) ||
            !ch::make_map(&maps.x[i], c.x, n_tok, c.k, c.ldx, ch::BN))
            return IB_ERR_UNSUPPORTED;
    }
    for (int i = n; i < ch::MAX_PHASES; ++i) { p.ph[i] = p.ph[0]; maps.w[i] = maps.w[0]; maps.x[i] = maps.x[0]; }
    constexpr size_t smem = (size_t)ch::STAGES * (ch::A_BYTES + ch::B_BYTES) + (2 * ch::STAGES + 5) * 8 + 5 * ch::SSQ_LD * 4 + 2 * ch::SLOT * 4 + 1024;
    static IbDeviceSet configured;
    if (const int e = ib_allow_dynamic_smem(configured, ch::chain_kernel, smem)) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(ch::THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeCooperative;     // its CTAs wait for each other: all of them must be resident
    attr[0].val.cooperative = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ch::g_pdl ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, ch::chain_kernel, maps, p);
    return e == cudaSuccess ? ib_launch_status() : (int)e;
}

IB_EXPORT void ib_gemm_chain_set_pdl(int on) { ch::g_pdl = on; }

IB_EXPORT int ib_gemm_chain_error(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, ch::g_error, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(ch::g_error, &zero, sizeof(int));
    }
    return v;
}

IB_EXPORT int ib_gemm_chain_error_async(int* out, cudaStream_t stream) {
    return (int)cudaMemcpyFromSymbolAsync(out, ch::g_error, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
}

#endif
