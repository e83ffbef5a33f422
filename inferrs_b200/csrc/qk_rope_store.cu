// Per-head RMSNorm of queries and keys, rotation by position, and the write of
// keys and values into their cache pages: one kernel, one pass over the fused
// projection output.
//
// Input row layout: [ n_heads*d queries | n_kv_heads*d keys | n_kv_heads*d values ]
// (or queries only, when the layer reads another entry's cache).
// Norm, rotation angle tables (float) and the products are all 32-bit; only the
// stores are act_t.
#include "common.cuh"

#define QRS_WARPS 4

// A row whose position lies outside the rotation tables is left out, and the first such row is recorded here
// (row + 1; 0: none) for the host to read with ib_row_fault.  A row whose page is not in the cache (-1 in the
// block table: a request that stands in to fill a batch) writes no key or value; that is no fault.
__device__ int ib_row_fault_word = 0;

__device__ __forceinline__ void ib_note_row_fault(int row) {
    if ((threadIdx.x & 31) == 0) atomicCAS(&ib_row_fault_word, 0, row + 1);
}

// The recorded fault (row + 1, 0 if none), or a negative cudaError_t; waits for the device.
IB_EXPORT int ib_row_fault(int reset) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, ib_row_fault_word, sizeof(int));
    if (e != cudaSuccess) return -(int)e;
    if (reset && v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(ib_row_fault_word, &zero, sizeof(int));
    }
    return v;
}

// The same word on its way to `out` (pinned host memory) in stream order, without waiting for the device.
IB_EXPORT int ib_row_fault_async(int* out, cudaStream_t stream) {
    return (int)cudaMemcpyFromSymbolAsync(out, ib_row_fault_word, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
}

// A request's last row of the step clears the places behind its value in the value's page.  The attention kernels
// that fetch whole pages give those places a probability of zero, but zero times what an earlier owner of the
// page may have left there (an infinity, no number at all) would not be zero.  Keys need no clearing: a score is
// replaced, not multiplied, where a key is not visible.
__device__ __forceinline__ bool ib_last_row_of_request(const int* __restrict__ row_request, int row, int n_rows) {
    return row + 1 >= n_rows || row_request[row + 1] != row_request[row];
}

template <typename WT>
__global__ void qk_norm_rope_store_kernel(
    const act_t* __restrict__ qkv, int row_stride, int n_heads, int n_kv_heads, int head_dim, int store_kv,
    const WT* __restrict__ q_weight, const WT* __restrict__ k_weight, float eps,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, int rot_dim, int interleaved, int table_rows,
    const int* __restrict__ positions, const int* __restrict__ row_request,
    const int* __restrict__ block_table, int max_pages, int page_size, int n_pages,
    act_t* __restrict__ k_pages, act_t* __restrict__ v_pages, act_t* __restrict__ q_out) {
    extern __shared__ float smem[];
    ib_grid_dependency_sync();
    const int row = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int d = head_dim;
    const int half = rot_dim / 2;
    float* sh = smem + warp * d;
    const int pos = positions[row];
    const int heads_total = n_heads + (store_kv ? 2 * n_kv_heads : 0);
    // a position outside the rotation tables: the row is left out and the fault is recorded
    if (pos < 0 || (rot_dim > 0 && pos >= table_rows)) { ib_note_row_fault(row); return; }

    // Where this row's key and value go: page and place within the page.
    long kv_base = -1;  // element offset of (page, kv head 0, slot, 0)
    if (store_kv) {
        const int req = row_request[row];
        const int page = pos / page_size < max_pages ? block_table[(long)req * max_pages + pos / page_size] : -1;
        if (page >= 0 && page < n_pages)
            kv_base = ((long)page * n_kv_heads * page_size + (pos % page_size)) * d;
    }
    const bool clear_tail = kv_base >= 0 && ib_last_row_of_request(row_request, row, gridDim.x);

    // one warp per head: blockIdx.y picks the group of QRS_WARPS heads
    for (int head = blockIdx.y * QRS_WARPS + warp; head < heads_total; head += heads_total) {
        const act_t* src = qkv + (long)row * row_stride + (long)head * d;
        const int kind = head < n_heads ? 0 : (head < n_heads + n_kv_heads ? 1 : 2);  // 0 q, 1 k, 2 v
        float ss = 0.0f;
        for (int j = lane; j < d; j += 32) {
            const float v = ib_to_float(src[j]);
            sh[j] = v;
            ss += v * v;
        }
        act_t* dst;
        if (kind == 0) {
            dst = q_out + ((long)row * n_heads + head) * d;
        } else {
            if (kv_base < 0) { __syncwarp(); continue; }
            const int kvh = head - n_heads - (kind == 2 ? n_kv_heads : 0);
            dst = (kind == 1 ? k_pages : v_pages) + kv_base + (long)kvh * page_size * d;
        }
        if (kind == 2) {
            for (int j = lane; j < d; j += 32) dst[j] = ib_from_float<act_t>(sh[j]);
            if (clear_tail) {
                const int behind = (page_size - 1 - pos % page_size) * d;
                for (int j = lane; j < behind; j += 32) dst[d + j] = ib_from_float<act_t>(0.0f);
            }
            __syncwarp();
            continue;
        }
        const WT* w = kind == 0 ? q_weight : k_weight;
        if (w != nullptr) {
            ss = ib_warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)d + eps);
            for (int j = lane; j < d; j += 32) sh[j] = sh[j] * inv * ib_to_float(w[j]);
        }
        __syncwarp();
        const float* c = cos_table + (long)pos * half;
        const float* s = sin_table + (long)pos * half;
        // element i of the first half turns with element i + rot_dim / 2, or (interleaved) element 2i with 2i + 1
        for (int j = lane; j < d; j += 32) {
            float o;
            if (j >= rot_dim) o = sh[j];
            else if (interleaved) o = (j & 1) ? sh[j - 1] * s[j >> 1] + sh[j] * c[j >> 1] : sh[j] * c[j >> 1] - sh[j + 1] * s[j >> 1];
            else if (j < half) o = sh[j] * c[j] - sh[j + half] * s[j];
            else o = sh[j - half] * s[j - half] + sh[j] * c[j - half];
            dst[j] = ib_from_float<act_t>(o);
        }
        __syncwarp();  // sh is overwritten by this warp's next head
    }
}

#if IB_ACT_BF16
// Head size 128 rotated in full, bfloat16: one warp per (row, HPW heads), lane l holds elements 4l..4l+3 of each
// head and gets the elements 64 further (or nearer) from lane l ^ 16; no shared memory.  All HPW loads are issued
// before the first is used: with thousands of rows the kernel is bound by the bytes it keeps in flight.
template <typename WT, int HPW>
__global__ void qk_norm_rope_store_d128_kernel(
    const __nv_bfloat16* __restrict__ qkv, int row_stride, int n_heads, int n_kv_heads, int store_kv,
    const WT* __restrict__ q_weight, const WT* __restrict__ k_weight, float eps,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, int table_rows,
    const int* __restrict__ positions, const int* __restrict__ row_request,
    const int* __restrict__ block_table, int max_pages, int page_size, int n_pages,
    __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ q_out) {
    // the step's description, the tables and the weights are written by no kernel: they are fetched while the
    // kernel before this one still runs; the projection's output only after it has finished
    ib_grid_dependency_launch();
    const int row = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = n_heads + (store_kv ? 2 * n_kv_heads : 0);
    const int head0 = (blockIdx.y * QRS_WARPS + warp) * HPW;
    if (head0 >= heads_total) return;
    const int pos = positions[row];
    if (pos < 0 || pos >= table_rows) { ib_note_row_fault(row); ib_grid_dependency_wait(); return; }
    long kv_base = -1;  // element offset of (page, kv head 0, place in the page, 0)
    if (store_kv && head0 + HPW > n_heads) {
        const int req = row_request[row];
        const int page = pos / page_size < max_pages ? block_table[(long)req * max_pages + pos / page_size] : -1;
        if (page >= 0 && page < n_pages) kv_base = ((long)page * n_kv_heads * page_size + (pos % page_size)) * 128;
    }
    const bool clear_tail = kv_base >= 0 && ib_last_row_of_request(row_request, row, gridDim.x);
    // element i < 64 pairs with i + 64: lanes 0..15 hold the first halves, lanes 16..31 the second
    const int i0 = 4 * (lane & 15);
    const float4 c = *reinterpret_cast<const float4*>(cos_table + (long)pos * 64 + i0);
    const float4 s = *reinterpret_cast<const float4*>(sin_table + (long)pos * 64 + i0);
    const float cs[4] = {c.x, c.y, c.z, c.w}, sn[4] = {s.x, s.y, s.z, s.w};
    float wq[4] = {1.0f, 1.0f, 1.0f, 1.0f}, wk[4] = {1.0f, 1.0f, 1.0f, 1.0f};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        if (q_weight != nullptr && head0 < n_heads) wq[e] = ib_to_float(q_weight[4 * lane + e]);
        if (k_weight != nullptr && head0 + HPW > n_heads) wk[e] = ib_to_float(k_weight[4 * lane + e]);
    }
    ib_grid_dependency_wait();
    uint2 raw[HPW];
#pragma unroll
    for (int h = 0; h < HPW; ++h)
        if (head0 + h < heads_total)
            raw[h] = *reinterpret_cast<const uint2*>(qkv + (long)row * row_stride + (long)(head0 + h) * 128 + 4 * lane);
#pragma unroll
    for (int h = 0; h < HPW; ++h) {
        const int head = head0 + h;
        if (head >= heads_total) break;
        const int kind = head < n_heads ? 0 : (head < n_heads + n_kv_heads ? 1 : 2);
        const float2 x01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[h].x));
        const float2 x23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[h].y));
        float x[4] = {x01.x, x01.y, x23.x, x23.y};
        __nv_bfloat16* dst;
        if (kind == 0) {
            dst = q_out + ((long)row * n_heads + head) * 128;
        } else {
            if (kv_base < 0) continue;
            const int kvh = head - n_heads - (kind == 2 ? n_kv_heads : 0);
            dst = (kind == 1 ? k_pages : v_pages) + kv_base + (long)kvh * page_size * 128;
        }
        if (kind != 2) {
            const WT* w = kind == 0 ? q_weight : k_weight;
            if (w != nullptr) {
                float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
                ss = ib_warp_sum(ss);
                const float inv = 1.0f / sqrtf(ss / 128.0f + eps);
#pragma unroll
                for (int e = 0; e < 4; ++e) x[e] = x[e] * inv * (kind == 0 ? wq[e] : wk[e]);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float other = __shfl_xor_sync(0xffffffffu, x[e], 16);
                x[e] = lane < 16 ? x[e] * cs[e] - other * sn[e] : other * sn[e] + x[e] * cs[e];
            }
        }
        uint2 o;
        *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(x[0], x[1]);
        *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(x[2], x[3]);
        *reinterpret_cast<uint2*>(dst + 4 * lane) = o;
        if (kind == 2 && clear_tail)
            for (int k = 1; k < page_size - pos % page_size; ++k)
                *reinterpret_cast<uint2*>(dst + k * 128 + 4 * lane) = make_uint2(0u, 0u);
    }
}
#endif

#if IB_ACT_BF16
// The same for thousands of rows, where bytes in flight and instructions per byte decide: sixteen lanes per
// head, each with four elements of the head's first half and the four that rotate with them in the second half
// (element i pairs with i + 64), so the rotation needs no exchange between lanes.  A warp takes two heads at a
// time and eight heads in all; all loads are issued before the first is used.
template <typename WT>
__global__ void qk_norm_rope_store_d128_wide_kernel(
    const __nv_bfloat16* __restrict__ qkv, int row_stride, int n_heads, int n_kv_heads, int store_kv,
    const WT* __restrict__ q_weight, const WT* __restrict__ k_weight, float eps,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, int table_rows,
    const int* __restrict__ positions, const int* __restrict__ row_request,
    const int* __restrict__ block_table, int max_pages, int page_size, int n_pages,
    __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ q_out) {
    constexpr int HPW = 8;                       // heads per warp
    ib_grid_dependency_launch();
    const int row = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = n_heads + (store_kv ? 2 * n_kv_heads : 0);
    const int head0 = (blockIdx.y * (blockDim.x >> 5) + warp) * HPW;
    if (head0 >= heads_total) return;
    const int pos = positions[row];
    if (pos < 0 || pos >= table_rows) { ib_note_row_fault(row); ib_grid_dependency_wait(); return; }
    long kv_base = -1;
    if (store_kv && head0 + HPW > n_heads) {
        const int req = row_request[row];
        const int page = pos / page_size < max_pages ? block_table[(long)req * max_pages + pos / page_size] : -1;
        if (page >= 0 && page < n_pages) kv_base = ((long)page * n_kv_heads * page_size + (pos % page_size)) * 128;
    }
    const bool clear_tail = kv_base >= 0 && ib_last_row_of_request(row_request, row, gridDim.x);
    const int sub = lane >> 4, l16 = lane & 15;  // which of the two heads of a pass, and the place in it
    const int e0 = 4 * l16;                      // this lane's elements e0 .. e0 + 3 and 64 + e0 .. 64 + e0 + 3
    const float4 cs = *reinterpret_cast<const float4*>(cos_table + (long)pos * 64 + e0);
    const float4 sn = *reinterpret_cast<const float4*>(sin_table + (long)pos * 64 + e0);
    float wq[8], wk[8];                          // norm weights of the two runs of four
    {
        const bool has_q = q_weight != nullptr && head0 < n_heads, has_k = k_weight != nullptr && head0 + HPW > n_heads;
        auto four = [&](const WT* w, int at, float* out4) {   // w[at .. at + 3], at a multiple of four
            if constexpr (sizeof(WT) == 2) {
                const uint2 v = *reinterpret_cast<const uint2*>(w + at);
                const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
                const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
                out4[0] = a.x; out4[1] = a.y; out4[2] = b.x; out4[3] = b.y;
            } else {
                const float4 v = *reinterpret_cast<const float4*>(w + at);
                out4[0] = v.x; out4[1] = v.y; out4[2] = v.z; out4[3] = v.w;
            }
        };
#pragma unroll
        for (int e = 0; e < 8; ++e) wq[e] = wk[e] = 1.0f;
        if (has_q) { four(q_weight, e0, wq); four(q_weight, 64 + e0, wq + 4); }
        if (has_k) { four(k_weight, e0, wk); four(k_weight, 64 + e0, wk + 4); }
    }
    ib_grid_dependency_wait();
    uint2 raw_lo[HPW / 2], raw_hi[HPW / 2];
#pragma unroll
    for (int j = 0; j < HPW / 2; ++j) {
        const int head = head0 + 2 * j + sub;
        if (head < heads_total) {
            const __nv_bfloat16* src = qkv + (long)row * row_stride + (long)head * 128 + e0;
            raw_lo[j] = *reinterpret_cast<const uint2*>(src);
            raw_hi[j] = *reinterpret_cast<const uint2*>(src + 64);
        }
    }
#pragma unroll
    for (int j = 0; j < HPW / 2; ++j) {
        const int head = head0 + 2 * j + sub;
        const bool live = head < heads_total;   // the other half of the warp may still have a head: no early exit
        const int kind = head < n_heads ? 0 : (head < n_heads + n_kv_heads ? 1 : 2);
        float x[8];                              // 0..3: first half, 4..7: their partners in the second half
        {
            const __nv_bfloat162* lo2 = reinterpret_cast<const __nv_bfloat162*>(&raw_lo[j]);
            const __nv_bfloat162* hi2 = reinterpret_cast<const __nv_bfloat162*>(&raw_hi[j]);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float2 a = live ? __bfloat1622float2(lo2[e]) : make_float2(0.0f, 0.0f);
                const float2 b = live ? __bfloat1622float2(hi2[e]) : make_float2(0.0f, 0.0f);
                x[2 * e] = a.x; x[2 * e + 1] = a.y;
                x[4 + 2 * e] = b.x; x[4 + 2 * e + 1] = b.y;
            }
        }
        const WT* w = kind == 0 ? q_weight : k_weight;
        float ss = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);   // over the head's sixteen lanes
        if (kind != 2 && w != nullptr) {
            // the reciprocal square root in one step (two units in the last place of float32): with thousands of rows
            // this kernel is bound by its instructions, and the result is rounded to bfloat16
            const float inv = rsqrtf(ss * (1.0f / 128.0f) + eps);
#pragma unroll
            for (int e = 0; e < 8; ++e) x[e] = x[e] * inv * (kind == 0 ? wq[e] : wk[e]);
        }
        if (kind != 2) {
            const float c[4] = {cs.x, cs.y, cs.z, cs.w}, s4[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float lo = x[e], hi = x[4 + e];
                x[e] = lo * c[e] - hi * s4[e];
                x[4 + e] = lo * s4[e] + hi * c[e];
            }
        }
        if (!live) continue;
        __nv_bfloat16* dst;
        if (kind == 0) {
            dst = q_out + ((long)row * n_heads + head) * 128;
        } else {
            if (kv_base < 0) continue;
            const int kvh = head - n_heads - (kind == 2 ? n_kv_heads : 0);
            dst = (kind == 1 ? k_pages : v_pages) + kv_base + (long)kvh * page_size * 128;
        }
        uint2 o_lo, o_hi;
        __nv_bfloat162 t;
        t = __floats2bfloat162_rn(x[0], x[1]); o_lo.x = *reinterpret_cast<unsigned*>(&t);
        t = __floats2bfloat162_rn(x[2], x[3]); o_lo.y = *reinterpret_cast<unsigned*>(&t);
        t = __floats2bfloat162_rn(x[4], x[5]); o_hi.x = *reinterpret_cast<unsigned*>(&t);
        t = __floats2bfloat162_rn(x[6], x[7]); o_hi.y = *reinterpret_cast<unsigned*>(&t);
        *reinterpret_cast<uint2*>(dst + e0) = o_lo;
        *reinterpret_cast<uint2*>(dst + 64 + e0) = o_hi;
        if (kind == 2 && clear_tail)
            for (int k = 1; k < page_size - pos % page_size; ++k) {
                *reinterpret_cast<uint2*>(dst + k * 128 + e0) = make_uint2(0u, 0u);
                *reinterpret_cast<uint2*>(dst + k * 128 + 64 + e0) = make_uint2(0u, 0u);
            }
    }
}
#endif

IB_EXPORT int ib_qk_norm_rope_store(const void* qkv, int row_stride, int n_rows, int n_heads, int n_kv_heads,
                                    int head_dim, int store_kv, const void* q_weight, const void* k_weight,
                                    int weight_is_f32, float eps, const float* cos_table, const float* sin_table,
                                    int rot_dim, int interleaved, int table_rows, const int* positions, const int* row_request,
                                    const int* block_table, int max_pages, int page_size, int n_pages,
                                    void* k_pages, void* v_pages, void* q_out, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (head_dim <= 0 || head_dim > 1024 || n_heads <= 0 || rot_dim < 0 || rot_dim > head_dim || (rot_dim & 1))
        return IB_ERR_ARGUMENT;
    if (store_kv && (n_kv_heads <= 0 || page_size <= 0 || max_pages <= 0)) return IB_ERR_ARGUMENT;
    if (rot_dim > 0 && (cos_table == nullptr || sin_table == nullptr || table_rows <= 0)) return IB_ERR_ARGUMENT;
    const size_t smem = (size_t)QRS_WARPS * head_dim * sizeof(float);
    const int heads_total = n_heads + (store_kv ? 2 * n_kv_heads : 0);
    const dim3 grid(n_rows, (heads_total + QRS_WARPS - 1) / QRS_WARPS);
#if IB_ACT_BF16
    if (head_dim == 128 && rot_dim == 128 && !interleaved && (row_stride % 4) == 0 && ((uintptr_t)qkv % 8) == 0 &&
        ((uintptr_t)cos_table % 16) == 0 && ((uintptr_t)sin_table % 16) == 0) {
#define IB_LAUNCH_D128(WT, HPW)                                                                                    \
    ib_launch(qk_norm_rope_store_d128_kernel<WT, HPW>, dim3(n_rows, (heads_total + QRS_WARPS * HPW - 1) / (QRS_WARPS * HPW)), \
              32 * QRS_WARPS, 0, stream, (const __nv_bfloat16*)qkv, row_stride, n_heads, n_kv_heads, store_kv,          \
              (const WT*)q_weight, (const WT*)k_weight, eps, cos_table, sin_table, table_rows, positions, row_request,  \
              block_table, max_pages, page_size, n_pages, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages,            \
              (__nv_bfloat16*)q_out)
        // few rows: one head per warp, for the shortest chain; many rows: eight heads per warp and sixteen bytes
        // per lane, for bytes in flight (the cache pages and the output must then be 16-byte aligned)
        if (n_rows >= 256 && (row_stride % 8) == 0 && ((uintptr_t)qkv % 16) == 0 && ((uintptr_t)q_out % 16) == 0 &&
            ((uintptr_t)q_weight % 16) == 0 && ((uintptr_t)k_weight % 16) == 0 &&
            (!store_kv || (((uintptr_t)k_pages % 16) == 0 && ((uintptr_t)v_pages % 16) == 0))) {
            int warps = (heads_total + 7) / 8;
            if (warps > 8) warps = 8;
            const dim3 wide_grid(n_rows, (heads_total + 8 * warps - 1) / (8 * warps));
#define IB_LAUNCH_WIDE(WT)                                                                                            \
    ib_launch(qk_norm_rope_store_d128_wide_kernel<WT>, wide_grid, 32 * warps, 0, stream, (const __nv_bfloat16*)qkv,   \
              row_stride, n_heads, n_kv_heads, store_kv, (const WT*)q_weight, (const WT*)k_weight, eps, cos_table,     \
              sin_table, table_rows, positions, row_request, block_table, max_pages, page_size, n_pages,               \
              (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, (__nv_bfloat16*)q_out)
            if (weight_is_f32) IB_LAUNCH_WIDE(float); else IB_LAUNCH_WIDE(__nv_bfloat16);
#undef IB_LAUNCH_WIDE
        } else if (n_rows >= 256) {
            if (weight_is_f32) IB_LAUNCH_D128(float, 4); else IB_LAUNCH_D128(__nv_bfloat16, 4);
        } else {
            if (weight_is_f32) IB_LAUNCH_D128(float, 1); else IB_LAUNCH_D128(__nv_bfloat16, 1);
        }
#undef IB_LAUNCH_D128
        return ib_launch_status();
    }
#endif
    if (weight_is_f32)
        ib_launch(qk_norm_rope_store_kernel<float>, grid, 32 * QRS_WARPS, smem, stream,
            (const act_t*)qkv, row_stride, n_heads, n_kv_heads, head_dim, store_kv, (const float*)q_weight,
            (const float*)k_weight, eps, cos_table, sin_table, rot_dim, interleaved, table_rows, positions, row_request, block_table,
            max_pages, page_size, n_pages, (act_t*)k_pages, (act_t*)v_pages, (act_t*)q_out);
    else
        ib_launch(qk_norm_rope_store_kernel<__nv_bfloat16>, grid, 32 * QRS_WARPS, smem, stream,
            (const act_t*)qkv, row_stride, n_heads, n_kv_heads, head_dim, store_kv, (const __nv_bfloat16*)q_weight,
            (const __nv_bfloat16*)k_weight, eps, cos_table, sin_table, rot_dim, interleaved, table_rows, positions, row_request,
            block_table,
            max_pages, page_size, n_pages, (act_t*)k_pages, (act_t*)v_pages, (act_t*)q_out);
    return ib_launch_status();
}
