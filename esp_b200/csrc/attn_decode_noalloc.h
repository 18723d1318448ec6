// esp_attn_decode_noalloc: split-key decode attention for callers that must not allocate.
//
// This entry point has no counterpart in the reference project (merely-made/esp); it exists for hosts
// that embed this library but cannot ask the CUDA runtime for memory at the moment they need attention:
// a process that handed every byte of the device to its own arena at start-up and runs with the
// allocator locked, a latency-bound loop in which cudaMalloc or cudaFree (both of which may wait for
// the device) are forbidden, or a plug-in that runs under a host's memory accounting and may only use
// buffers the host passes in.  Such a caller still passes its inputs and its output; what it cannot
// provide is the scratch that the split-key kernel needs between its two passes.
//
// The scratch therefore lives inside the library: a file-scope __device__ array of
// ESP_ATTN_DECODE_NOALLOC_FLOATS floats (8 MiB) that every device which loads this library holds until
// the process exits.  The function calls neither cudaMalloc nor cudaFree nor any routine that allocates.
//
// Set-up: the first call on a device (with that device current) looks up the array's device address
// with cudaGetSymbolAddress and keeps it; make that first call before any stream capture begins.
// Limits: n_tokens * nh * n_splits * (hd + 2) must not exceed esp_attn_decode_noalloc_capacity() (the
// array less the ESP_NOALLOC_COUNTERS words kept for the kernel's counters) and n_tokens * nh must not
// exceed ESP_NOALLOC_COUNTERS, else the call returns ESP_NOALLOC_TOO_LARGE and launches nothing.  hd is
// 64, 128, 192 or 256 and split a multiple of 64, as for esp_attn_decode.
// Sharing: all calls on a device use the same array.  It keeps whatever the last call left there.  The
// kernel writes every partial result it later reads, so that part needs no clearing; the counters at
// the array's end must be zero when a call starts: they are zero when the library is loaded and each
// call puts them back to zero before it ends, also when one of its bounded waits runs out (such a block
// still takes part in its row's count, with an empty partial result, and the status word says so).  Two
// calls whose kernels can overlap on the GPU (different streams, no ordering between them) race on the
// array: order them.  On the host the entry point keeps its per-device address table without a lock:
// make the first call on each device from one thread.
//
// Arguments and result are those of esp_attn_decode without the two scratch pointers; the return value
// is 0, a cudaError_t, or ESP_NOALLOC_TOO_LARGE.
#pragma once
#include <cuda_runtime.h>

#define ESP_ATTN_DECODE_NOALLOC_FLOATS (2u << 20)
#define ESP_NOALLOC_COUNTERS 65536
#define ESP_NOALLOC_TOO_LARGE (-2)

#ifdef __cplusplus
extern "C" {
#endif

__attribute__((visibility("default"))) int esp_attn_decode_noalloc(
    const void* q, const void* k_cache, const void* v_cache, void* out, const int* tok_seq, const int* tok_pos,
    const int* block_table, int table_stride, int n_pages, int page, int n_tokens, int nh, int nkv, int hd, int window,
    int split, int n_splits, int* status, cudaStream_t stream);

// Number of floats of the built-in scratch that partial results may use (the limit the call checks against).
__attribute__((visibility("default"))) long long esp_attn_decode_noalloc_capacity(void);

#ifdef __cplusplus
}
#endif
