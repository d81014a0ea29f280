// Paged GQA decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference framework.  It exists for hosts that
// drive the kernels from a context where cudaMalloc is off limits: a plug-in that runs inside
// another runtime's memory budget, a latency-critical loop that must not touch the allocator, a
// process whose device memory is fully handed out up front.  Such a caller still passes its own
// inputs and the output buffer; what it cannot provide is the scratch that split-KV decoding needs
// for the per-split partial results.  Here that scratch is a fixed array inside the library.
//
//   int llb_gqa_decode_no_alloc(q, q_stride, kv_layer, req_to_token, r2t_stride, b_req_idx, b_seq_len,
//                               out, out_stride, B, Hq, Hkv, D, num_splits, sm_scale, stream);
//
// Same arguments and result as llb_gqa_decode without the two scratch pointers.
//
// Limits and rules
//   * The head size D must be 64 or 128 (any other value returns LLB_ERR_UNSUPPORTED, as the regular entry
//     point does).
//   * With num_splits > 1, B * Hq * num_splits must not exceed LLB_NO_ALLOC_MAX_ROWS (8192); a larger request
//     returns LLB_ERR_TOO_LARGE (-3) and launches nothing.  With num_splits == 1 the kernel writes the output
//     directly, the scratch is not touched and B * Hq may be any size.
//   * The scratch is (8192 * 128 + 8192) floats = 4 MiB + 32 KiB.  It is part of the library image, so
//     every GPU that loads the library keeps these bytes until the process exits.
//   * The first call on a device looks up the device address of the array (cudaGetSymbolAddress, with
//     that device current) and caches it.  Make that first call outside of any stream capture.
//   * The function never calls cudaMalloc, cudaFree or any allocating library routine.
//   * All calls share the one array and it keeps what the previous call left in it.  The kernels do
//     not rely on zeroed scratch (each split writes its slot or marks it empty), so nothing is cleared
//     between calls; but two calls that overlap on the GPU (different streams, or graphs replayed
//     concurrently) race on it.  Serialise them.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define LLB_NO_ALLOC_MAX_ROWS 8192

#ifdef __cplusplus
extern "C" {
#endif

int llb_gqa_decode_no_alloc(const void* q, int64_t q_stride, const void* kv_layer, const int* req_to_token,
                            int64_t r2t_stride, const int* b_req_idx, const int* b_seq_len, void* out,
                            int64_t out_stride, int B, int Hq, int Hkv, int D, int num_splits, float sm_scale,
                            cudaStream_t stream);

#ifdef __cplusplus
}
#endif
