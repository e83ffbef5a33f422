// y[n, m] = sum_k x[n, k] * w[m, k]   (weights stored [out, in], no bias)
//
// A plain FFMA kernel: no tensor cores, no reduced-precision mode.  Every output
// element is one chain of fused multiply-adds over k in ascending order, so its
// value does not depend on how many rows the batch has or where the row stands in
// it.  This is the matrix product of the true 32-bit path; with other element types
// it also serves 32-bit weights met by bfloat16 activations.
#include "common.cuh"

#define GT_BM 64
#define GT_BN 64
#define GT_BK 16

template <typename XT, typename WT, typename OT>
__global__ void __launch_bounds__(256) gemm_tn_simt_kernel(const XT* __restrict__ x, const WT* __restrict__ w,
                                                            OT* __restrict__ y, int n_rows, int n_out, int k_dim,
                                                            long ldx, long ldw, long ldy) {
    __shared__ float xs[GT_BK][GT_BM + 4];
    __shared__ float ws[GT_BK][GT_BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int row0 = blockIdx.y * GT_BM, col0 = blockIdx.x * GT_BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < k_dim; k0 += GT_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 256;
            const int r = idx >> 4, kk = idx & 15;
            const int gr = row0 + r, gc = col0 + r, gk = k0 + kk;
            xs[kk][r] = (gr < n_rows && gk < k_dim) ? ib_to_float(x[(long)gr * ldx + gk]) : 0.0f;
            ws[kk][r] = (gc < n_out && gk < k_dim) ? ib_to_float(w[(long)gc * ldw + gk]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GT_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gr = row0 + ty * 4 + i;
        if (gr >= n_rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gc = col0 + tx * 4 + j;
            if (gc < n_out) y[(long)gr * ldy + gc] = ib_from_float<OT>(acc[i][j]);
        }
    }
}

template <typename XT, typename WT, typename OT>
static int launch_gemm(const void* x, const void* w, void* y, int n_rows, int n_out, int k_dim, long ldx, long ldw,
                       long ldy, cudaStream_t stream) {
    const dim3 grid((n_out + GT_BN - 1) / GT_BN, (n_rows + GT_BM - 1) / GT_BM);
    gemm_tn_simt_kernel<XT, WT, OT><<<grid, 256, 0, stream>>>((const XT*)x, (const WT*)w, (OT*)y, n_rows, n_out,
                                                             k_dim, ldx, ldw, ldy);
    return ib_launch_status();
}

// x is act_t or float (x_is_f32), w is bfloat16 or float (w_is_f32), y is act_t or float (y_is_f32).
IB_EXPORT int ib_gemm_tn_simt(const void* x, int x_is_f32, const void* w, int w_is_f32, void* y, int y_is_f32,
                              int n_rows, int n_out, int k_dim, long ldx, long ldw, long ldy, cudaStream_t stream) {
    if (n_rows <= 0 || n_out <= 0) return IB_OK;
    if (k_dim <= 0) return IB_ERR_ARGUMENT;
#define IB_GEMM_CASE(XF, WF, YF, XT, WT, OT)                              \
    if ((x_is_f32 != 0) == XF && (w_is_f32 != 0) == WF && (y_is_f32 != 0) == YF) \
        return launch_gemm<XT, WT, OT>(x, w, y, n_rows, n_out, k_dim, ldx, ldw, ldy, stream);
    IB_GEMM_CASE(true, true, true, float, float, float)
#if IB_ACT_BF16
    IB_GEMM_CASE(false, false, false, act_t, __nv_bfloat16, act_t)
    IB_GEMM_CASE(false, false, true, act_t, __nv_bfloat16, float)
    IB_GEMM_CASE(false, true, false, act_t, float, act_t)
    IB_GEMM_CASE(false, true, true, act_t, float, float)
    IB_GEMM_CASE(true, true, false, float, float, act_t)
#endif
#undef IB_GEMM_CASE
    return IB_ERR_UNSUPPORTED;
}
