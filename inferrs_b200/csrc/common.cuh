// Shared helpers of the sm_100a kernels: element types, conversions, reductions, launch checks.
//
// Every library is built twice from the same sources: with -DIB_ACT_BF16=0 the
// activation and cache element `act_t` is float (the true 32-bit path), with
// -DIB_ACT_BF16=1 it is __nv_bfloat16.  Arithmetic inside the kernels is float in
// both builds; only what is stored between kernels changes.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#ifndef IB_ACT_BF16
#error "build with -DIB_ACT_BF16=0 or -DIB_ACT_BF16=1"
#endif

#if IB_ACT_BF16
typedef __nv_bfloat16 act_t;
#else
typedef float act_t;
#endif

#define IB_EXPORT extern "C" __attribute__((visibility("default")))

// Error codes returned by the exported functions.  0 is success; positive values are
// cudaError_t of the launch; negative values are refusals of the arguments.
#define IB_OK 0
#define IB_ERR_UNSUPPORTED (-1)
#define IB_ERR_ARGUMENT (-2)

__device__ __forceinline__ float ib_to_float(float v) { return v; }
__device__ __forceinline__ float ib_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T ib_from_float(float v);
template <> __device__ __forceinline__ float ib_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 ib_from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float ib_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float ib_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The order of
// the additions depends only on blockDim, so a row's result does not depend on the batch.
__device__ __forceinline__ float ib_block_sum(float v, float* smem32) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = ib_warp_sum(v);
    __syncthreads();  // smem32 may still be read from an earlier call
    if (lane == 0) smem32[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? smem32[lane] : 0.0f;
    r = ib_warp_sum(r);
    return r;
}

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch.  When the library's switch is on (ib_set_pdl), kernels are launched so
// that they may start before the kernel before them in the stream has finished.  Every kernel of this
// package therefore begins with ib_grid_dependency_sync(): it lets the kernel after it start in turn and
// then waits until the kernel before it has completed and its writes are visible.  Only what no kernel
// writes (weights, tables) may be read before that call.  With the switch off, or for a kernel launched
// the plain way, both instructions do nothing.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void ib_grid_dependency_sync() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// The two halves on their own, for kernels that fetch what no kernel writes (weights, tables, the step's
// description) between them.
__device__ __forceinline__ void ib_grid_dependency_launch() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void ib_grid_dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

extern int ib_pdl_enabled;  // one per library, defined beside its exported setter ib_set_pdl

template <typename... KArgs, typename... Args>
static inline void ib_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ib_pdl_enabled ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Dynamic shared memory beyond 48 KB has to be allowed per kernel and per device.  `done` remembers the devices
// of this process on which a kernel has it already (one bit each; a device beyond the 64th is set every time).
// Setting it twice is harmless, so two threads that meet here need no lock.
struct IbDeviceSet { std::atomic<unsigned long long> bits{0}; };

template <typename Kernel>
static inline int ib_allow_dynamic_smem(IbDeviceSet& done, Kernel kernel, size_t bytes) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    const bool tracked = dev >= 0 && dev < 64;
    if (tracked && ((done.bits.load(std::memory_order_acquire) >> dev) & 1ull)) return IB_OK;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return (int)e;
    if (tracked) done.bits.fetch_or(1ull << dev, std::memory_order_release);
    return IB_OK;
}

static inline int ib_launch_status() {
    cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? IB_OK : (int)e;
}
