// y[t, f] = sum_k x[t, k] * w[f, k]  as one persistent CTA per SM that streams an equal share of W.
//
// The work is cut into units of one 128x64 block of W (with the matching BNx64 block of x).  The units of
// all output tiles form one line, tile after tile, k-block after k-block, and CTA c takes the c-th equal
// slice of that line, whatever the shape of the product: every SM reads the same number of bytes, and
// the TMA ring never drains at a tile's edge.  A slice that begins or ends inside a tile yields a partial
// sum (float32, in a workspace with two slots per CTA).  The CTA that holds the tile's last k-blocks
// finishes the tile, after it has streamed all of its own slice: it waits for the flags of the CTAs that
// hold the tile's earlier k-blocks, adds the partial sums in the order of the CTAs and stores y.  Sums
// are therefore in a fixed order for a given shape: the same inputs give the same bits.
//
// Per CTA: warp 0 = TMA producer, warp 1 = MMA issuer (tcgen05.mma, two accumulators in tensor memory so
// that the epilogue of one slice overlaps the MMAs of the next), warps 2..5 = epilogue.
//
// All waits are bounded (about two seconds): mbarrier waits, and the finisher's wait for flags.  A wait
// that runs out records a code in the library's error word; the CTA then lets copies in flight land,
// frees its tensor memory and returns.  A finisher only ever waits for CTAs with a lower index.
#include <cuda.h>

#include "common.cuh"
#include "sm100.cuh"

#if IB_ACT_BF16

namespace sk {

using namespace sm100;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int A_BYTES = BM * BK * 2;

__device__ int g_error = 0;

// a bounded wait that reports through this file's error word
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, int code) {
    return mbar_wait_bounded(bar, parity, &g_error, code);
}

__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }  // warps 2..5
__device__ __forceinline__ int ld_acquire(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release(int* p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

struct Params {
    void* y;
    float* partial;   // [grid][2][BN * BM] float32, column (token) major: a tail and a head partial sum per CTA
    int* flags;       // [grid], zero between launches
    long ldy;
    int n_tok, n_out, num_kb, tiles_f, n_tiles, y_is_f32;
    long total_units;
};

// first unit of CTA c's slice
__device__ __forceinline__ long slice_begin(long total, int grid, int c) { return total * c / grid; }

template <int BN, int STAGES>
__global__ void __launch_bounds__(THREADS, 1) streamk_kernel(const __grid_constant__ CUtensorMap map_w,
                                                             const __grid_constant__ CUtensorMap map_x, const Params p) {
    constexpr int B_BYTES = BN * BK * 2;
    constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
    extern __shared__ unsigned char raw_smem[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~(uintptr_t)1023);
    unsigned char* a_tiles = smem;
    unsigned char* b_tiles = smem + STAGES * A_BYTES;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(b_tiles + STAGES * B_BYTES);
    const unsigned full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const unsigned accf0 = smem_u32(bars + 2 * STAGES), acce0 = smem_u32(bars + 2 * STAGES + 2);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * STAGES + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cta = blockIdx.x, grid = gridDim.x;
    const long u0 = slice_begin(p.total_units, grid, cta), u1 = slice_begin(p.total_units, grid, cta + 1);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(accf0 + 8 * b, 1); mbar_init(acce0 + 8 * b, 4); }
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

    if (warp == 0) {
        if (lane == 0) {
            long i = 0;
            for (long u = u0; u < u1; ++u, ++i) {
                const int s = (int)(i % STAGES);
                if (i >= STAGES && !mbar_wait(empty0 + 8 * s, (unsigned)((i / STAGES) - 1) & 1, 1)) { ok = false; break; }
                const int tile = (int)(u / p.num_kb), kb = (int)(u - (long)tile * p.num_kb);
                const int tile_t = tile / p.tiles_f, tile_f = tile - tile_t * p.tiles_f;
                mbar_expect_tx(full0 + 8 * s, A_BYTES + B_BYTES);
                tma_load_2d(smem_u32(a_tiles + s * A_BYTES), &map_w, kb * BK, tile_f * BM, full0 + 8 * s);
                tma_load_2d(smem_u32(b_tiles + s * B_BYTES), &map_x, kb * BK, tile_t * BN, full0 + 8 * s);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
            long i = 0;
            int seg = 0;
            bool first = true;  // the next MMA starts a slice of a tile
            for (long u = u0; u < u1 && ok; ++u, ++i) {
                const int s = (int)(i % STAGES);
                const int kb = (int)(u % p.num_kb);
                const int buf = seg & 1;
                if (first && seg >= 2 && !mbar_wait(acce0 + 8 * buf, (unsigned)((seg >> 1) - 1) & 1, 4)) { ok = false; break; }
                if (!mbar_wait(full0 + 8 * s, (unsigned)(i / STAGES) & 1, 2)) { ok = false; break; }
                fence_after();
                const unsigned long long da = desc_k_major(smem_u32(a_tiles + s * A_BYTES));
                const unsigned long long db = desc_k_major(smem_u32(b_tiles + s * B_BYTES));
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    umma(tmem + buf * BN, da + (unsigned long long)(k * UMMA_K * 2 / 16),
                         db + (unsigned long long)(k * UMMA_K * 2 / 16), idesc, (first && k == 0) ? 0u : 1u);
                first = false;
                umma_commit(empty0 + 8 * s);
                if (kb == p.num_kb - 1 || u == u1 - 1) {  // the slice of this tile ends here
                    umma_commit(accf0 + 8 * buf);
                    ++seg;
                    first = true;
                }
            }
        }
    } else {
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const bool leader = threadIdx.x == 64;  // first thread of the epilogue warps
        float* tail = p.partial + (long)cta * 2 * BN * BM;   // partial sum of a slice that does not end its tile
        float* head = tail + BN * BM;                        // partial sum of a slice that ends a tile begun by others
        int head_tile = -1;
        int seg = 0;
        for (long u = u0; u < u1 && ok; ++seg) {
            const int tile = (int)(u / p.num_kb);
            const int kb_begin = (int)(u - (long)tile * p.num_kb);
            const long tile_end = (long)(tile + 1) * p.num_kb;
            const long seg_end = tile_end < u1 ? tile_end : u1;
            const bool ends_tile = seg_end == tile_end;
            const int tile_t = tile / p.tiles_f, tile_f = tile - tile_t * p.tiles_f;
            const int feature = tile_f * BM + row;
            const int buf = seg & 1;
            if (!__all_sync(0xffffffffu, mbar_wait(accf0 + 8 * buf, (unsigned)(seg >> 1) & 1, 3))) { ok = false; break; }  // warp-wide
            fence_after();
            // a slice that covers its whole tile is stored; any other is kept as a partial sum
            float* keep = !ends_tile ? tail : (kb_begin > 0 ? head : nullptr);
            if (keep == head) head_tile = tile;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                float v[16];
                tmem_ld16(tmem + ((unsigned)(q * 32) << 16) + buf * BN + c0, v);
                if (keep != nullptr) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) keep[(c0 + j) * BM + row] = v[j];
                } else if (feature < p.n_out) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int tok = tile_t * BN + c0 + j;
                        if (tok < p.n_tok) {
                            if (p.y_is_f32) reinterpret_cast<float*>(p.y)[(long)tok * p.ldy + feature] = v[j];
                            else reinterpret_cast<__nv_bfloat16*>(p.y)[(long)tok * p.ldy + feature] = __float2bfloat16_rn(v[j]);
                        }
                    }
                }
            }
            fence_before();
            if (lane == 0) mbar_arrive(acce0 + 8 * buf);  // this warp has read the accumulator
            if (keep == tail) {
                __threadfence();
                epilogue_sync();                           // all four warps have written their part
                if (leader) st_release(p.flags + cta, 1);  // the CTA that finishes this tile may read it
            }
            u = seg_end;
        }
        // Finish the tile whose last k-blocks were this CTA's first slice.  This comes last, so that no CTA's
        // stream of W waits for another CTA: the partial sums it needs are written when their CTAs are done
        // streaming, which is about now.
        if (head_tile >= 0 && ok) {
            const long tile_begin = (long)head_tile * p.num_kb;
            int first_c = (int)(tile_begin * grid / p.total_units);
            while (first_c > 0 && slice_begin(p.total_units, grid, first_c) > tile_begin) --first_c;
            while (slice_begin(p.total_units, grid, first_c + 1) <= tile_begin) ++first_c;
            if (leader) {
                const unsigned long long t0 = global_ns();
                bool waiting = true;
                for (int c = first_c; c < cta && waiting; ++c) {
                    unsigned it = 0;
                    while (ld_acquire(p.flags + c) == 0) {
                        if ((++it & 255u) == 0 && global_ns() - t0 > 2000000000ull) {
                            atomicCAS(&g_error, 0, 5);
                            waiting = false;
                            break;
                        }
                    }
                }
            }
            epilogue_sync();
            const int tile_t = head_tile / p.tiles_f, tile_f = head_tile - tile_t * p.tiles_f;
            const int feature = tile_f * BM + row;
            if (feature < p.n_out) {
#pragma unroll 1
                for (int c0 = 0; c0 < BN && tile_t * BN + c0 < p.n_tok; c0 += 16) {
                    float v[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = 0.0f;
                    for (int c = first_c; c < cta; ++c) {   // in the order of the CTAs, then this CTA's own part
                        const float* theirs = p.partial + (long)c * 2 * BN * BM + c0 * BM + row;
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] += __ldcg(theirs + j * BM);
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int tok = tile_t * BN + c0 + j;
                        if (tok < p.n_tok) {
                            const float sum = v[j] + head[(c0 + j) * BM + row];
                            if (p.y_is_f32) reinterpret_cast<float*>(p.y)[(long)tok * p.ldy + feature] = sum;
                            else reinterpret_cast<__nv_bfloat16*>(p.y)[(long)tok * p.ldy + feature] = __float2bfloat16_rn(sum);
                        }
                    }
                }
            }
            epilogue_sync();                               // all four warps have read the partial sums
            if (leader)
                for (int c = first_c; c < cta; ++c) p.flags[c] = 0;  // zero again for the next launch
        }
    }

    if (!ok || g_error != 0) {
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
static int launch(const CUtensorMap& mw, const CUtensorMap& mx, const Params& p, int grid, cudaStream_t stream) {
    constexpr size_t smem = (size_t)STAGES * (A_BYTES + BN * BK * 2) + (2 * STAGES + 6) * 8 + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(streamk_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    streamk_kernel<BN, STAGES><<<grid, THREADS, smem, stream>>>(mw, mx, p);
    return ib_launch_status();
}

}  // namespace sk

// Floats of workspace that a product with `n_tok` tokens needs for `grid` CTAs (plus `grid` ints of flags).
IB_EXPORT long ib_gemm_streamk_workspace_floats(int n_tok, int grid) {
    const int bn = n_tok <= 16 ? 16 : n_tok <= 32 ? 32 : n_tok <= 64 ? 64 : n_tok <= 128 ? 128 : 256;
    return (long)grid * 2 * bn * sk::BM;
}

// x [n_tok, k], w [n_out, k] bfloat16 (row strides ldx, ldw); y [n_tok, n_out] bfloat16 or float32.
// partial: ib_gemm_streamk_workspace_floats(n_tok, grid) floats; flags: grid ints that are zero (the kernel
// leaves them zero).  grid: number of persistent CTAs, at most one per SM.  Launches that share a
// workspace must not overlap.
IB_EXPORT int ib_gemm_tn_streamk(const void* x, long ldx, const void* w, long ldw, void* y, long ldy, int y_is_f32,
                                 int n_tok, int n_out, int k, float* partial, int* flags, int grid,
                                 cudaStream_t stream) {
    if (n_tok <= 0 || n_out <= 0) return IB_OK;
    if (k <= 0 || grid <= 0 || partial == nullptr || flags == nullptr) return IB_ERR_ARGUMENT;
    if ((k % 8) || (ldx % 8) || (ldw % 8) || ((uintptr_t)x % 16) || ((uintptr_t)w % 16)) return IB_ERR_UNSUPPORTED;
    const int bn = n_tok <= 16 ? 16 : n_tok <= 32 ? 32 : n_tok <= 64 ? 64 : n_tok <= 128 ? 128 : 256;
    sk::Params p;
    p.y = y; p.partial = partial; p.flags = flags; p.ldy = ldy; p.n_tok = n_tok; p.n_out = n_out;
    p.num_kb = (k + sk::BK - 1) / sk::BK;
    p.tiles_f = (n_out + sk::BM - 1) / sk::BM;
    p.n_tiles = p.tiles_f * ((n_tok + bn - 1) / bn);
    p.y_is_f32 = y_is_f32;
    p.total_units = (long)p.n_tiles * p.num_kb;
    if (grid > p.total_units) grid = (int)p.total_units;
    CUtensorMap mw, mx;
    if (!sk::make_map(&mw, w, n_out, k, ldw, sk::BM) || !sk::make_map(&mx, x, n_tok, k, ldx, bn)) return IB_ERR_UNSUPPORTED;
    switch (bn) {
        case 16: return sk::launch<16, 10>(mw, mx, p, grid, stream);
        case 32: return sk::launch<32, 9>(mw, mx, p, grid, stream);
        case 64: return sk::launch<64, 8>(mw, mx, p, grid, stream);
        case 128: return sk::launch<128, 6>(mw, mx, p, grid, stream);
        default: return sk::launch<256, 4>(mw, mx, p, grid, stream);
    }
}

IB_EXPORT int ib_gemm_streamk_error(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, sk::g_error, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(sk::g_error, &zero, sizeof(int));
    }
    return v;
}

#endif
