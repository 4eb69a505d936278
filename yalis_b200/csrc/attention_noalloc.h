// Split-key decode attention without any allocation by the callee or the caller's framework.
//
// This entry point has no counterpart in axonn-ai/yalis (whose attention is a library call
// that allocates through PyTorch).  It exists for host programs that drive this library
// through its C symbols and must not allocate device memory once they are running: for
// example a serving process that hands all device memory to its own arena at start-up, so a
// later cudaMalloc can fail although memory is "free" inside the arena, or a loop with a
// latency budget in which cudaMalloc's implicit device-wide synchronisation is not
// acceptable.  Such a caller still owns its inputs and its output; what it cannot provide
// is the temporary memory the split-key kernel needs between its two phases.
//
// yalis_paged_attention_mma_noalloc() is yalis_paged_attention_mma() (see attention_mma.cu)
// with that temporary memory taken from a fixed array that is part of the loaded library:
//
//   * the array is YALIS_NOALLOC_SCRATCH_BYTES (16 MiB + 64 KiB) of device memory per GPU,
//     held by every GPU on which the library's module is loaded, from load until exit;
//   * a call needs  n_requests * kv_heads * 4  bytes of counters (at most 64 KiB) and
//     n_tokens * heads * n_splits * (head_dim + 2) * 4  bytes of partial results (at most
//     16 MiB); a larger problem is refused with YALIS_ERR_SCRATCH (-5) and nothing is
//     launched (yalis_paged_attention_mma_noalloc_needed() tells the size beforehand);
//   * the first call on a device looks up the array's device address once
//     (cudaGetSymbolAddress, with that device current).  Make this first call outside any
//     stream capture; later calls on that device do no set-up;
//   * every call on a device uses the same array.  The counters are cleared on the
//     caller's stream before each launch and whatever else the array holds from earlier
//     calls is overwritten before it is read, but two calls whose kernels can run at the
//     same time on one GPU (different streams, no ordering between them) race on it: order
//     such calls yourself;
//   * no cudaMalloc, cudaFree or allocating library routine is called, in the first call or
//     later.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#define YALIS_NOALLOC_TICKET_BYTES (64 * 1024)
#define YALIS_NOALLOC_PARTIAL_BYTES (16 * 1024 * 1024)
#define YALIS_NOALLOC_SCRATCH_BYTES (YALIS_NOALLOC_TICKET_BYTES + YALIS_NOALLOC_PARTIAL_BYTES)
#define YALIS_ERR_SCRATCH (-5)

#ifdef __cplusplus
extern "C" {
#endif

// Bytes of the fixed array that a call with these sizes would use: counters (rounded into the
// first 64 KiB) and partial results.  Compare with the two limits above.
__attribute__((visibility("default"))) long long yalis_paged_attention_mma_noalloc_needed(
    int n_tokens, int n_requests, int nh, int g, int hs, int n_splits, long long* ticket_bytes,
    long long* partial_bytes);

// Same arguments and result codes as yalis_paged_attention_mma, without `scratch` and `tickets`.
// Returns YALIS_ERR_SCRATCH if the problem does not fit the fixed array.
__attribute__((visibility("default"))) int yalis_paged_attention_mma_noalloc(
    const void* q, int q_stride, void* out, int out_stride, const void* k_pool, const void* v_pool,
    const int32_t* positions, const int32_t* q_start, const int32_t* req_of_token, const int32_t* block_table,
    int table_width, int page_size, int num_pages, int n_tokens, int n_requests, int max_q_len, int nh, int g,
    int hs, float scale, int window, int n_splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
