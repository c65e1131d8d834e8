// Decode attention for callers that are not allowed to allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for
// embedders of this library.
//
// Who needs it: code that runs where cudaMalloc is off limits -- a plugin inside
// a host process that hands out a fixed memory budget up front, a real-time loop
// that must not take the allocator's lock (cudaMalloc may synchronise the whole
// device), or a process that already filled the GPU and cannot get another byte.
// The regular entry point (slb_decode_attention_bf16) needs a scratch buffer for
// the partial results of its key splits, which somebody has to allocate.  This
// variant brings its own: a fixed array that is part of the library image.
//
// Contract
//   * Inputs and outputs are passed exactly as for slb_decode_attention_bf16
//     (num_pages is the number of pages in k_cache / v_cache; a block-table entry
//     outside [0, num_pages) is read as zeros and reported by slb_attention_status),
//     minus the scratch pointer.  Nothing is allocated or freed: no cudaMalloc,
//     no cudaFree, no library routine that allocates.
//   * The scratch is a file-scope device array of
//     slb_decode_attention_noalloc_capacity_bytes() bytes (4 MiB).  Every GPU on
//     which this library is loaded keeps that much memory until the process ends.
//   * A call needs S * H * num_splits * (head_dim + 2) * 4 bytes of it.  Larger
//     requests are refused with SLB_ERR_TOO_LARGE (-2) and nothing is launched;
//     slb_decode_attention_noalloc_strerror() gives the reason as text.
//   * The first call on a device looks up the array's device address (once per
//     device, with that device current).  Make that first call before any stream
//     capture begins.
//   * All calls share the one array and it keeps what the last call left.  Nothing
//     in it has to start at zero: every slot the combine step reads is written by
//     the split kernel of the same call.  That also holds for a block that gives up
//     one of its bounded waits: it marks its slots as empty, so the combine step never
//     merges an earlier call's leftovers; the result of that head then lacks those
//     keys, and slb_attention_status() is non-zero -- check it where a wrong result
//     must not pass silently.  Two calls that overlap on the GPU (other streams, other
//     threads) race on the array; run them one after the other.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

int slb_decode_attention_bf16_noalloc(const __nv_bfloat16* q, int ldq, const __nv_bfloat16* k_cache,
                                      const __nv_bfloat16* v_cache, __nv_bfloat16* out, int ldo,
                                      const int* block_table, int max_pages, const int* ctx_len,
                                      int S, int H, int Hkv, int page_size, int num_pages, float scale,
                                      int window, int num_splits, cudaStream_t stream);

long long slb_decode_attention_noalloc_capacity_bytes(void);

const char* slb_decode_attention_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
