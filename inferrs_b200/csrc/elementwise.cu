// Embedding gather, fused residual-add + RMSNorm, SiLU-gate product.
//
// The residual stream is float in both builds: the sum x + delta is formed and
// kept in 32-bit, and only the normalised copy that feeds the next matrix
// product is stored as act_t.
#include "common.cuh"

int ib_pdl_enabled = 0;

// 1: the kernels of this library are launched so that they may start before their predecessor in the stream
// has finished (see common.cuh); 0: plain stream order.
IB_EXPORT void ib_set_pdl(int on) { ib_pdl_enabled = on; }

// ---------------------------------------------------------------------------
// Embedding: out[row, :] = table[ids[row], :] * scale   (the product is formed in float32; scale 1 for
// architectures that do not scale their embeddings)
// ---------------------------------------------------------------------------
template <typename WT>
__global__ void embedding_gather_kernel(const WT* __restrict__ table, const int* __restrict__ ids,
                                        float* __restrict__ out, int width, int vocab, float scale) {
    ib_grid_dependency_sync();
    const int row = blockIdx.x;
    const int id = ids[row];
    const bool ok = id >= 0 && id < vocab;  // the host refuses such ids before the launch
    const WT* src = table + (size_t)(ok ? id : 0) * width;
    float* dst = out + (size_t)row * width;
    for (int j = threadIdx.x; j < width; j += blockDim.x) dst[j] = ok ? ib_to_float(src[j]) * scale : 0.0f;
}

IB_EXPORT int ib_embedding_gather(const void* table, int table_is_f32, const int* ids, float* out, int n_rows,
                                  int width, int vocab, float scale, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (width <= 0 || vocab <= 0) return IB_ERR_ARGUMENT;
    const int threads = width >= 1024 ? 256 : 128;
    if (table_is_f32)
        ib_launch(embedding_gather_kernel<float>, n_rows, threads, 0, stream, (const float*)table, ids, out, width, vocab,
                  scale);
    else
        ib_launch(embedding_gather_kernel<__nv_bfloat16>, n_rows, threads, 0, stream, (const __nv_bfloat16*)table, ids, out,
                  width, vocab, scale);
    return ib_launch_status();
}

// ---------------------------------------------------------------------------
// Token ids that are still on the device: ids[i] < 0 stands for carry[-1 - ids[i]], the token that an
// earlier step sampled and the host has not read yet.  Runs in the stream before the step that reads ids.
// ---------------------------------------------------------------------------
__global__ void resolve_tokens_kernel(int* __restrict__ ids, int n, const int* __restrict__ carry, int n_carry) {
    ib_grid_dependency_sync();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int v = ids[i];
    if (v < 0) {
        const int src = -1 - v;
        ids[i] = src < n_carry ? carry[src] : -1;   // the embedding gives zeros for an id that is no token
    }
}

IB_EXPORT int ib_resolve_tokens(int* ids, int n, const int* carry, int n_carry, cudaStream_t stream) {
    if (n <= 0) return IB_OK;
    if (n_carry < 0 || (n_carry > 0 && carry == nullptr)) return IB_ERR_ARGUMENT;
    ib_launch(resolve_tokens_kernel, (n + 255) / 256, 256, 0, stream, ids, n, carry, n_carry);
    return ib_launch_status();
}

// ---------------------------------------------------------------------------
// x += delta (kept in the float residual), out = x / sqrt(mean(x^2) + eps) * w
//
// rows == nullptr : row r of residual/delta -> row r of out; the sum is written back.
// rows != nullptr : row rows[r] of residual/delta -> row r of out; nothing is written
//                   back (used for the last norm, which only the wanted rows need).
// ---------------------------------------------------------------------------
template <typename WT>
__global__ void add_rms_norm_kernel(float* __restrict__ residual, const act_t* __restrict__ delta,
                                    const WT* __restrict__ weight, act_t* __restrict__ out,
                                    const int* __restrict__ rows, int width, float eps) {
    __shared__ float red[32];
    ib_grid_dependency_sync();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* res = residual + (size_t)src * width;
    const act_t* del = delta ? delta + (size_t)src * width : nullptr;
    const bool write_back = (rows == nullptr) && (del != nullptr);
    float ss = 0.0f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        float v = res[j];
        if (del) v += ib_to_float(del[j]);
        if (write_back) res[j] = v;
        ss += v * v;
    }
    ss = ib_block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    act_t* dst = out + (size_t)r * width;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        float v = res[j];  // this thread's own write, if there was one
        if (del && !write_back) v += ib_to_float(del[j]);
        dst[j] = ib_from_float<act_t>(v * inv * ib_to_float(weight[j]));
    }
}

// Four elements per thread and step (16-byte loads of the residual), for widths that are multiples of 4 and
// at most 4 * NORM_KEEP * (threads per block).
#define NORM_KEEP 4
struct alignas(8) ActVec4 { act_t v[4]; };
template <typename WT> struct alignas(sizeof(WT) * 4) WVec4 { WT v[4]; };

template <typename WT>
__global__ void add_rms_norm_vec4_kernel(float* __restrict__ residual, const act_t* __restrict__ delta,
                                         const WT* __restrict__ weight, act_t* __restrict__ out,
                                         const int* __restrict__ rows, int width, float eps) {
    __shared__ float red[32];
    ib_grid_dependency_launch();
    const int n4 = width >> 2;
    // the norm's weights are fetched while the kernel before this one still runs
    const WVec4<WT>* w4 = reinterpret_cast<const WVec4<WT>*>(weight);
    WVec4<WT> wk[NORM_KEEP];
#pragma unroll
    for (int k = 0; k < NORM_KEEP; ++k) {
        const int j = threadIdx.x + k * blockDim.x;
        if (j < n4) wk[k] = w4[j];
    }
    ib_grid_dependency_wait();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float4* res = reinterpret_cast<float4*>(residual + (size_t)src * width);
    const ActVec4* del = delta ? reinterpret_cast<const ActVec4*>(delta + (size_t)src * width) : nullptr;
    const bool write_back = (rows == nullptr) && (del != nullptr);
    // the row stays in registers between the two passes (the host picks a block size that makes it fit)
    float4 keep[NORM_KEEP];
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < NORM_KEEP; ++k) {
        const int j = threadIdx.x + k * blockDim.x;
        if (j < n4) {
            float4 v = res[j];
            if (del) {
                const ActVec4 d = del[j];
                v.x += ib_to_float(d.v[0]); v.y += ib_to_float(d.v[1]);
                v.z += ib_to_float(d.v[2]); v.w += ib_to_float(d.v[3]);
            }
            if (write_back) res[j] = v;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            keep[k] = v;
        }
    }
    ss = ib_block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    ActVec4* dst = reinterpret_cast<ActVec4*>(out + (size_t)r * width);
#pragma unroll
    for (int k = 0; k < NORM_KEEP; ++k) {
        const int j = threadIdx.x + k * blockDim.x;
        if (j >= n4) break;
        const float4 v = keep[k];
        const WVec4<WT> w = wk[k];
        ActVec4 o;
        o.v[0] = ib_from_float<act_t>(v.x * inv * ib_to_float(w.v[0]));
        o.v[1] = ib_from_float<act_t>(v.y * inv * ib_to_float(w.v[1]));
        o.v[2] = ib_from_float<act_t>(v.z * inv * ib_to_float(w.v[2]));
        o.v[3] = ib_from_float<act_t>(v.w * inv * ib_to_float(w.v[3]));
        dst[j] = o;
    }
}

static inline bool ib_aligned16(const void* p) { return p == nullptr || ((uintptr_t)p & 15) == 0; }

IB_EXPORT int ib_add_rms_norm(float* residual, const void* delta, const void* weight, int weight_is_f32, void* out,
                              const int* rows, int n_rows, int width, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (width <= 0) return IB_ERR_ARGUMENT;
    int threads = 128;
    if (width >= 2048) threads = 512;
    else if (width >= 512) threads = 256;
    if ((width & 3) == 0 && width <= 4 * NORM_KEEP * 1024 && ib_aligned16(residual) && ib_aligned16(delta) &&
        ib_aligned16(weight) && ib_aligned16(out)) {
        int t4 = 128;   // enough threads that NORM_KEEP float4 per thread hold the row
        while (4 * NORM_KEEP * t4 < width) t4 <<= 1;
        if (width >= 4096 && t4 < 256) t4 = 256;
        if (weight_is_f32)
            ib_launch(add_rms_norm_vec4_kernel<float>, n_rows, t4, 0, stream, residual, (const act_t*)delta,
                      (const float*)weight, (act_t*)out, rows, width, eps);
        else
            ib_launch(add_rms_norm_vec4_kernel<__nv_bfloat16>, n_rows, t4, 0, stream, residual, (const act_t*)delta,
                      (const __nv_bfloat16*)weight, (act_t*)out, rows, width, eps);
        return ib_launch_status();
    }
    if (weight_is_f32)
        ib_launch(add_rms_norm_kernel<float>, n_rows, threads, 0, stream, residual, (const act_t*)delta,
                  (const float*)weight, (act_t*)out, rows, width, eps);
    else
        ib_launch(add_rms_norm_kernel<__nv_bfloat16>, n_rows, threads, 0, stream, residual, (const act_t*)delta,
                  (const __nv_bfloat16*)weight, (act_t*)out, rows, width, eps);
    return ib_launch_status();
}

// ---------------------------------------------------------------------------
// A norm on a sub-layer's output (before it is added to the residual stream): out = x / sqrt(mean(x^2) + eps) * w
// for rows of act_t.  And the form of the fused kernel above for a sub-layer without a norm: x += delta, out = x
// as act_t.
// ---------------------------------------------------------------------------
template <typename WT>
__global__ void rms_norm_rows_kernel(const act_t* __restrict__ x, const WT* __restrict__ weight,
                                     act_t* __restrict__ out, int width, float eps) {
    __shared__ float red[32];
    ib_grid_dependency_sync();
    const act_t* src = x + (size_t)blockIdx.x * width;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        const float v = ib_to_float(src[j]);
        ss += v * v;
    }
    ss = ib_block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    act_t* dst = out + (size_t)blockIdx.x * width;
    for (int j = threadIdx.x; j < width; j += blockDim.x)
        dst[j] = ib_from_float<act_t>(ib_to_float(src[j]) * inv * ib_to_float(weight[j]));
}

IB_EXPORT int ib_rms_norm_rows(const void* x, const void* weight, int weight_is_f32, void* out, int n_rows, int width,
                               float eps, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (width <= 0 || weight == nullptr) return IB_ERR_ARGUMENT;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    if (weight_is_f32)
        ib_launch(rms_norm_rows_kernel<float>, n_rows, threads, 0, stream, (const act_t*)x, (const float*)weight,
                  (act_t*)out, width, eps);
    else
        ib_launch(rms_norm_rows_kernel<__nv_bfloat16>, n_rows, threads, 0, stream, (const act_t*)x,
                  (const __nv_bfloat16*)weight, (act_t*)out, width, eps);
    return ib_launch_status();
}

__global__ void add_cast_kernel(float* __restrict__ residual, const act_t* __restrict__ delta, act_t* __restrict__ out,
                                const int* __restrict__ rows, int width) {
    ib_grid_dependency_sync();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* res = residual + (size_t)src * width;
    const act_t* del = delta ? delta + (size_t)src * width : nullptr;
    act_t* dst = out + (size_t)r * width;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        float v = res[j];
        if (del) v += ib_to_float(del[j]);
        if (del && rows == nullptr) res[j] = v;
        dst[j] = ib_from_float<act_t>(v);
    }
}

IB_EXPORT int ib_add_cast(float* residual, const void* delta, void* out, const int* rows, int n_rows, int width,
                          cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (width <= 0) return IB_ERR_ARGUMENT;
    ib_launch(add_cast_kernel, n_rows, width >= 1024 ? 256 : 128, 0, stream, residual, (const act_t*)delta, (act_t*)out,
              rows, width);
    return ib_launch_status();
}

// ---------------------------------------------------------------------------
// What some architectures do to their logits, in place on float32: x *= scale, then, with cap > 0,
// x = cap * tanh(x / cap).
// ---------------------------------------------------------------------------
__global__ void logit_scale_softcap_kernel(float* __restrict__ logits, long total, float scale, float cap) {
    ib_grid_dependency_sync();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        float v = logits[i] * scale;
        if (cap > 0.0f) v = cap * tanhf(v / cap);
        logits[i] = v;
    }
}

IB_EXPORT int ib_logit_scale_softcap(float* logits, long total, float scale, float cap, cudaStream_t stream) {
    if (total <= 0) return IB_OK;
    long blocks = (total + 255) / 256;
    if (blocks > 148L * 16) blocks = 148L * 16;
    ib_launch(logit_scale_softcap_kernel, (int)blocks, 256, 0, stream, logits, total, scale, cap);
    return ib_launch_status();
}

// ---------------------------------------------------------------------------
// out[r, j] = silu(gate_up[r, j]) * gate_up[r, inner + j],  silu(z) = z / (1 + exp(-z))
// ---------------------------------------------------------------------------
__global__ void silu_gate_kernel(const act_t* __restrict__ gate_up, act_t* __restrict__ out, int inner, long total) {
    ib_grid_dependency_sync();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long r = i / inner;
        const int j = (int)(i - r * inner);
        const float g = ib_to_float(gate_up[r * 2 * inner + j]);
        const float u = ib_to_float(gate_up[r * 2 * inner + inner + j]);
        out[i] = ib_from_float<act_t>(g / (1.0f + expf(-g)) * u);
    }
}

#if IB_ACT_BF16
// Eight bfloat16 (16 bytes) per thread, for inner sizes that are multiples of 8: one row per blockIdx.y, so no
// thread divides to find its row.  With thousands of rows this kernel is bound by its instructions, not by
// memory, if exponential and division are the exact ones (about twenty instructions per element); the results
// are rounded to bfloat16, so the fast forms (ex2- and rcp-based, two units in the last place of float32) give
// the same bits but for a rare tie.
__global__ void silu_gate_vec8_kernel(const act_t* __restrict__ gate_up, act_t* __restrict__ out, int inner) {
    ib_grid_dependency_sync();
    const int in8 = inner >> 3;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= in8) return;
    const long r = blockIdx.y;
    const uint4 g = reinterpret_cast<const uint4*>(gate_up + r * 2 * inner)[j];
    const uint4 u = reinterpret_cast<const uint4*>(gate_up + r * 2 * inner + inner)[j];
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint4 o;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 gv = __bfloat1622float2(gp[k]), uv = __bfloat1622float2(up[k]);
        op[k] = __floats2bfloat162_rn(__fdividef(gv.x, 1.0f + __expf(-gv.x)) * uv.x,
                                      __fdividef(gv.y, 1.0f + __expf(-gv.y)) * uv.y);
    }
    reinterpret_cast<uint4*>(out + r * inner)[j] = o;
}
#endif

// Four elements per thread and step, for inner sizes that are multiples of 4.
__global__ void silu_gate_vec4_kernel(const act_t* __restrict__ gate_up, act_t* __restrict__ out, int inner, long total4) {
    ib_grid_dependency_sync();
    const int in4 = inner >> 2;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (long)gridDim.x * blockDim.x) {
        const long r = i / in4;
        const int j = (int)(i - r * in4);
        const ActVec4 g = reinterpret_cast<const ActVec4*>(gate_up + r * 2 * inner)[j];
        const ActVec4 u = reinterpret_cast<const ActVec4*>(gate_up + r * 2 * inner + inner)[j];
        ActVec4 o;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float gv = ib_to_float(g.v[k]);
            o.v[k] = ib_from_float<act_t>(gv / (1.0f + expf(-gv)) * ib_to_float(u.v[k]));
        }
        reinterpret_cast<ActVec4*>(out + r * inner)[j] = o;
    }
}

IB_EXPORT int ib_silu_gate(const void* gate_up, void* out, int n_rows, int inner, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (inner <= 0) return IB_ERR_ARGUMENT;
    const long total = (long)n_rows * inner;
#if IB_ACT_BF16
    if ((inner & 7) == 0 && ib_aligned16(gate_up) && ib_aligned16(out)) {
        const int in8 = inner >> 3;
        const int threads = in8 >= 256 ? 256 : ((in8 + 31) / 32) * 32;
        for (int r0 = 0; r0 < n_rows; r0 += 65535) {   // blockIdx.y holds at most 65,535 rows
            const int rows = n_rows - r0 < 65535 ? n_rows - r0 : 65535;
            ib_launch(silu_gate_vec8_kernel, dim3((in8 + threads - 1) / threads, rows), threads, 0, stream,
                      (const act_t*)gate_up + (long)r0 * 2 * inner, (act_t*)out + (long)r0 * inner, inner);
        }
        return ib_launch_status();
    }
#endif
    if ((inner & 3) == 0 && ib_aligned16(gate_up) && ib_aligned16(out)) {
        const long total4 = total >> 2;
        long b4 = (total4 + 255) / 256;
        if (b4 > 148L * 32) b4 = 148L * 32;
        ib_launch(silu_gate_vec4_kernel, (int)b4, 256, 0, stream, (const act_t*)gate_up, (act_t*)out, inner, total4);
        return ib_launch_status();
    }
    long blocks = (total + 255) / 256;
    if (blocks > 148L * 16) blocks = 148L * 16;
    ib_launch(silu_gate_kernel, (int)blocks, 256, 0, stream, (const act_t*)gate_up, (act_t*)out, inner, total);
    return ib_launch_status();
}

// ---------------------------------------------------------------------------
// Casts between float and act_t (used where a 32-bit weight meets bfloat16 activations).
// ---------------------------------------------------------------------------
__global__ void act_to_float_kernel(const act_t* __restrict__ in, float* __restrict__ out, long total) {
    ib_grid_dependency_sync();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x)
        out[i] = ib_to_float(in[i]);
}

IB_EXPORT int ib_act_to_float(const void* in, float* out, long total, cudaStream_t stream) {
    if (total <= 0) return IB_OK;
    long blocks = (total + 255) / 256;
    if (blocks > 148L * 16) blocks = 148L * 16;
    ib_launch(act_to_float_kernel, (int)blocks, 256, 0, stream, (const act_t*)in, out, total);
    return ib_launch_status();
}
