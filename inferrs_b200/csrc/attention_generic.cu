// Grouped-query attention over the paged cache, for any head size: one warp per
// (token, query head), 32-bit arithmetic throughout.
//
// A token at position `pos` of its request sees the keys lo..pos of that request,
// lo = 0 or pos - window + 1.  This step's keys are already in the cache when the
// kernel runs, so a prompt portion and a decoded token are the same case.  Keys are
// taken 32 at a time in ascending order from a multiple of 32, with an online
// softmax; the order of every sum depends only on (pos, window), never on what else
// is in the batch or on which pages hold the keys.
//
// This is the kernel of the true 32-bit path and the fallback of the bfloat16 path
// for head sizes that its tensor-core kernels do not take.
#include "common.cuh"

#define ATT_WARPS 4

template <int DPL>  // head-size elements per lane: head_dim <= 32 * DPL
__global__ void paged_attention_generic_kernel(
    const act_t* __restrict__ q, const act_t* __restrict__ k_pages, const act_t* __restrict__ v_pages,
    const int* __restrict__ block_table, int max_pages, int page_size, int n_pages,
    const int* __restrict__ row_request, const int* __restrict__ positions, int n_heads, int n_kv_heads,
    int head_dim, float scale, int window, act_t* __restrict__ out) {
    extern __shared__ float smem[];
    ib_grid_dependency_sync();
    const int row = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * ATT_WARPS + warp;
    if (head >= n_heads) return;  // whole warps leave; only warp-level syncs follow
    const int d = head_dim;
    float* qs = smem + warp * d;
    const int pos = positions[row];
    const int req = row_request[row];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int kvh = head / (n_heads / n_kv_heads);
    const int* bt = block_table + (long)req * max_pages;

    const act_t* qr = q + ((long)row * n_heads + head) * d;
    for (int e = lane; e < d; e += 32) qs[e] = ib_to_float(qr[e]);
    __syncwarp();

    float acc[DPL];
#pragma unroll
    for (int k = 0; k < DPL; ++k) acc[k] = 0.0f;
    float m = -INFINITY, l = 0.0f;

    for (int j0 = (lo / 32) * 32; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j >= lo && j <= pos;
        float s = -INFINITY;
        long off = 0;
        if (valid) {
            const int page = bt[j / page_size];
            if (page >= 0 && page < n_pages) {
                off = (((long)page * n_kv_heads + kvh) * page_size + (j % page_size)) * d;
                const act_t* kr = k_pages + off;
                float dot = 0.0f;
                for (int e = 0; e < d; ++e) dot = fmaf(qs[e], ib_to_float(kr[e]), dot);
                s = dot * scale;
            }
        }
        const float m_new = fmaxf(m, ib_warp_max(s));
        const float p = (s == -INFINITY) ? 0.0f : expf(s - m_new);
        const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
        l = l * corr + ib_warp_sum(p);
#pragma unroll
        for (int k = 0; k < DPL; ++k) acc[k] *= corr;
        const int n_in_chunk = (pos - j0 + 1 < 32) ? pos - j0 + 1 : 32;
        for (int jj = 0; jj < n_in_chunk; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long voff = __shfl_sync(0xffffffffu, off, jj);
            if (pj == 0.0f) continue;  // masked key (uniform over the warp)
            const act_t* vr = v_pages + voff;
#pragma unroll
            for (int k = 0; k < DPL; ++k) {
                const int e = lane + 32 * k;
                if (e < d) acc[k] = fmaf(pj, ib_to_float(vr[e]), acc[k]);
            }
        }
        m = m_new;
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    act_t* dst = out + ((long)row * n_heads + head) * d;
#pragma unroll
    for (int k = 0; k < DPL; ++k) {
        const int e = lane + 32 * k;
        if (e < d) dst[e] = ib_from_float<act_t>(acc[k] * inv);
    }
}

IB_EXPORT int ib_paged_attention_generic(const void* q, const void* k_pages, const void* v_pages,
                                         const int* block_table, int max_pages, int page_size, int n_pages,
                                         const int* row_request, const int* positions, int n_rows, int n_heads,
                                         int n_kv_heads, int head_dim, float scale, int window, void* out,
                                         cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads || head_dim <= 0 || page_size <= 0 || max_pages <= 0)
        return IB_ERR_ARGUMENT;
    if (head_dim > 512) return IB_ERR_UNSUPPORTED;
    const dim3 grid(n_rows, (n_heads + ATT_WARPS - 1) / ATT_WARPS);
    const size_t smem = (size_t)ATT_WARPS * head_dim * sizeof(float);
#define IB_LAUNCH_ATT(DPL)                                                                                      \
    ib_launch(paged_attention_generic_kernel<DPL>, grid, 32 * ATT_WARPS, smem, stream,                          \
        (const act_t*)q, (const act_t*)k_pages, (const act_t*)v_pages, block_table, max_pages, page_size,       \
        n_pages, row_request, positions, n_heads, n_kv_heads, head_dim, scale, window, (act_t*)out)
    if (head_dim <= 32) IB_LAUNCH_ATT(1);
    else if (head_dim <= 64) IB_LAUNCH_ATT(2);
    else if (head_dim <= 128) IB_LAUNCH_ATT(4);
    else if (head_dim <= 256) IB_LAUNCH_ATT(8);
    else IB_LAUNCH_ATT(16);
#undef IB_LAUNCH_ATT
    return ib_launch_status();
}
