// Declaration of the one entry point of this library that allocates no memory at all.
//
// It has no counterpart in the reference (ericcurtin/inferrs): the reference allocates a tensor for
// every intermediate result.  It exists for hosts that cannot let a library allocate device memory
// while it serves requests:
//   * a server that has given every byte the GPU had left to its pool of cache pages, so that a
//     later cudaMalloc could fail in the middle of a request;
//   * a process whose device memory belongs to an arena or allocator of its own with a fixed
//     budget, which must not be bypassed;
//   * a loop that must not stall: cudaMalloc and cudaFree may synchronise the whole device.
//
// The regular entry point, ib_paged_attention_mma in its decode form with more than one split, is
// given two scratch buffers by its caller (the Python layer allocates them for every call).  This
// variant does the same work with scratch that is part of the library image: a file-scope
// `static __device__` array of IB_NOALLOC_SCRATCH_FLOATS floats (16 MiB).  Every GPU on which the
// library is loaded holds those 16 MiB from load until the process exits.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Capacity of the built-in scratch.  A call needs n_rows * n_heads * n_splits * (head_dim + 2) floats.
#define IB_NOALLOC_SCRATCH_FLOATS (4 * 1024 * 1024)

// Return codes: 0 success; > 0 a cudaError_t; the negative ones below.
#define IB_NOALLOC_ERR_UNSUPPORTED (-1)  // head_dim not 64/128/256, page size does not divide 64, > 16 heads per kv head
#define IB_NOALLOC_ERR_ARGUMENT (-2)     // a size is zero or negative, or heads are not a multiple of kv heads
#define IB_NOALLOC_ERR_TOO_LARGE (-3)    // the call needs more scratch than IB_NOALLOC_SCRATCH_FLOATS
#define IB_NOALLOC_ERR_BUILD (-4)        // the library was built without the bfloat16 kernels

// Attention of one new token per request over its paged keys and values (bfloat16), the keys of
// every request cut `n_splits` ways and merged.  Same arithmetic, same results as
// ib_paged_attention_mma(..., decode_form = 1, n_splits, part_o, part_ml).
//
//   q            [n_rows, n_heads, head_dim] bfloat16, row r is request r's new token
//   k_pages, v_pages  [n_pages, n_kv_heads, page_size, head_dim] bfloat16
//   block_table  [n_rows, max_pages] int32 page ids of each request
//   row_request  [n_rows] int32, row_request[r] = r;   q_start [n_rows + 1] int32, q_start[r] = r
//   positions    [n_rows] int32 position of each new token (its key is already in the cache)
//   out          [n_rows, n_heads * head_dim] bfloat16
//
// It calls no cudaMalloc, cudaFree or other allocating routine.  The first call on a device looks
// up the device address of the built-in scratch (cudaGetSymbolAddress, with that device current),
// allows the kernel its dynamic shared memory on that device, and keeps both per device; make
// that first call before any stream capture begins on that device.
//
// All calls on a device share the one scratch array.  Nothing in it has to start at zero (every
// cell that is read has been written by the same call), and what a call leaves there is of no use
// to the next.  Two calls that overlap on the GPU (different streams, no dependency) race on it:
// order them.
int ib_paged_attention_decode_noalloc(const void* q, const void* k_pages, const void* v_pages,
                                      const int* block_table, int max_pages, int page_size, int n_pages,
                                      const int* row_request, const int* q_start, const int* positions,
                                      int n_rows, int n_heads, int n_kv_heads, int head_dim, float scale,
                                      int window, void* out, int n_splits, cudaStream_t stream);

// A sentence for a return code of the function above.
const char* ib_paged_attention_decode_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
