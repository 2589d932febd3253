// Split-KV decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in jason-fxz/mini-sglang (its attention comes from library
// wheels that allocate their own work buffers); it is an addition of this engine.
//
// Who needs it: code that runs where a device allocation is not possible or not allowed at call
// time -- a serving process whose memory budget was handed out completely at start-up (weights,
// cache pool), so that a late cudaMalloc fails; a host application that forbids allocator calls on
// its request path because cudaMalloc and cudaFree may synchronise the whole device; a plugin that
// is given raw pointers and a stream and nothing else.  The regular entry point, msgl_attention,
// expects the caller to bring scratch memory for the partial results of the kv splits; this one
// brings its own: a file-scope `static __device__` array inside the library.
//
// What the caller must know:
//   * The scratch array holds MSGL_NOALLOC_SCRATCH_FLOATS floats (16 MiB).  Every GPU that loads
//     the library keeps that much memory occupied until the process exits, whether or not this
//     function is ever called.
//   * A call needs max_split * B * n_q * (d + 2) floats.  Larger problems are refused with
//     MSGL_ERR_SCRATCH (5); nothing is launched then.  Use msgl_attention with your own scratch.
//   * The first call on each device does that device's set-up, with the device current: it looks
//     up the array's device address (cudaGetSymbolAddress) and raises the kernels' limit of
//     dynamic shared memory (cudaFuncSetAttribute), and remembers both per device.  Make that
//     first call during set-up, before any stream capture, with the problem shapes you will use
//     later (a group of more than 16 query heads per kv head takes another kernel than a small
//     one); later calls on the device do no set-up work.
//   * The function calls no cudaMalloc, cudaFree or any other allocating routine.
//   * All calls share the one array, and it keeps what the last call left in it.  Nothing in it
//     has to start at zero: every value a call reads was written earlier by that same call (each
//     split block writes its partial sums, maxima and row sums before the merge reads them).
//     Two calls that overlap on the GPU (different streams, no ordering between them) race on
//     the array and give wrong results; keep calls on one stream or order them with events.
//
// Shapes: one new token per request (decode).  q, out: [B, n_q, d] bfloat16 or float32 (dtype 1 / 0);
// k_cache, v_cache: [pages][n_kv][page_size][d]; q_start: [B + 1] = 0..B; kv_len: [B] tokens in the
// cache including the new one; block_table: [B, bt_stride]; nsplit: [B], each 1..max_split.
// Returns 0 when the kernels were launched, else one of the MSGL_ERR_* codes of common.cuh or 5.
#pragma once
#include <cuda_runtime.h>

#define MSGL_NOALLOC_SCRATCH_FLOATS (4u * 1024u * 1024u)
#define MSGL_ERR_SCRATCH 5

#ifdef __cplusplus
extern "C" {
#endif

int msgl_attention_decode_noalloc(const void* q, void* out, const void* k_cache, const void* v_cache,
                                  const int* q_start, const int* kv_len, const int* block_table, const int* nsplit,
                                  int B, int n_q, int n_kv, int d, int page_size, int bt_stride, int window,
                                  int max_split, float scale, int dtype, cudaStream_t stream);

// the stated maximum, for callers that want to check before they call
unsigned long long msgl_attention_noalloc_capacity_floats(void);

#ifdef __cplusplus
}
#endif
