// rf_attention_decode_noalloc: decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in maeddesg/ROCmForge; it exists for this library's users only.
//
// Who needs it: code that runs where cudaMalloc is off limits.  Examples are a callback inside
// someone else's serving loop that owns all device memory and hands out only tensor pointers, a
// host thread that must never take the allocator's lock (a real-time or signal-adjacent path),
// or a process that has deliberately given all remaining device memory to a cache and wants no
// later allocation to fail.  Such callers can still pass inputs and outputs they already own,
// but they cannot provide or request the kernel's scratch space (per-chunk partial results and
// arrival counters).  Here that scratch lives in a fixed array inside the library's own device
// image, so a call allocates nothing: no cudaMalloc, no cudaFree, no allocating library routine.
//
// Limits and rules:
//   * The array is RF_NOALLOC_SCRATCH_BYTES (8 MiB) and is held by every GPU that loads this
//     library until the process ends.  A call whose scratch need
//         B * heads * max_chunks * (head_dim + 2) * 4  +  B * kv_heads * 4   bytes
//     exceeds it is refused with RF_ERR_UNSUPPORTED (-2) and does nothing.
//   * The first call on a device looks the array's device address up (cudaGetSymbolAddress) with
//     that device current.  Make this first call outside any CUDA stream capture.
//   * All calls share the one array, and it keeps what the previous call left.  The arrival
//     counters are cleared at the start of every call (on the given stream); the rest is fully
//     rewritten before it is read.  Two calls that overlap on the GPU (different streams without
//     an ordering between them) race on the array: order them.
//   * max_chunks must cover the longest sequence of the call: ceil(length / 128) chunks, counted from
//     position 0 also for a layer with a window (partials are indexed by absolute chunk).  The lengths
//     live on the device, so the host cannot check this; a sequence that needs more chunks is left
//     alone by the kernel (its output rows stay as they were) and the status word is set to 3.
//   * Same arguments and same result as rf_attention_decode, without its three scratch pointers.
//     Returns 0, a cudaError_t (> 0), or RF_ERR_BAD_ARG (-1) / RF_ERR_UNSUPPORTED (-2).
#pragma once
#include <cuda_runtime.h>

#define RF_NOALLOC_SCRATCH_BYTES (8u << 20)

#ifdef __cplusplus
extern "C" {
#endif

int rf_attention_decode_noalloc(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                const void* v_pages, const int* tok_seq, const int* tok_pos, const int* seq_slot,
                                const int* block_table, int max_pages, int nh, int nkv, int hd, float scale,
                                int window, int B, int max_chunks, int* status, cudaStream_t st);

#ifdef __cplusplus
}
#endif
