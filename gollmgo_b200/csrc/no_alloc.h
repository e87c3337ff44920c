// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in TensorGreed/gollmgo; it is an addition
// of this library.
//
// Who it is for: code that runs where cudaMalloc is off limits -- a plug-in
// inside a host program that owns the device's memory budget, a real-time loop
// that must not hit the allocator, a thin C binding without torch's caching
// allocator behind it.  gg_attn_decode needs two scratch buffers from its caller
// (the per-slice partial outputs and their max/sum pairs).  This variant keeps
// that scratch inside the library, in one fixed array in device memory, so the
// caller passes inputs and outputs only.
//
// Limits and rules:
//   * The scratch array is GG_NOALLOC_SCRATCH_BYTES (about 4.3 MB).  Every GPU on
//     which this library is loaded holds it until the process exits.
//   * A call needs n_dec * nh * num_splits * d floats of partial outputs (at most
//     GG_NOALLOC_MAX_PART_O) and n_dec * nh * num_splits * 2 floats of max/sum
//     pairs (at most GG_NOALLOC_MAX_PART_ML); a larger call is refused with
//     GG_ERR_INVALID and a message, nothing is launched.
//   * The first call on a device looks up the array's device address (once per
//     device, with that device current).  Make that first call outside of any
//     stream capture.  Host threads may make their first calls at the same time:
//     the cached address is an atomic, and all of them find the same one.
//   * Arguments are checked before anything else; a call that is refused has
//     touched neither the device nor the array.
//   * All calls share the one array, and it keeps whatever the last call left in
//     it.  Nothing in it has to start at zero: each call writes every entry it
//     later reads.  Two calls that overlap on the GPU (different streams, no
//     dependency between them) race on the array; order them.
//   * It calls no cudaMalloc, cudaFree or any allocating library routine.
#pragma once
#include <cuda_runtime.h>

#define GG_NOALLOC_MAX_PART_O (1 << 20)      /* floats */
#define GG_NOALLOC_MAX_PART_ML (1 << 16)     /* floats */
#define GG_NOALLOC_SCRATCH_BYTES ((GG_NOALLOC_MAX_PART_O + GG_NOALLOC_MAX_PART_ML) * 4)

#ifdef __cplusplus
extern "C" {
#endif
// Same arguments and result as gg_attn_decode, without part_o and part_ml.
int gg_attn_decode_noalloc(const void* q, long long q_stride, const void* kcache,
                           const void* vcache, int dtype, const int* block_tables, int bt_stride,
                           const int* cu_q_lens, const int* context_lens, const int* dec_seqs,
                           int n_dec, int num_splits, void* out, int nh, int nkv, int d,
                           int page_size, int window, float scale, int allow_mma,
                           cudaStream_t stream);
#ifdef __cplusplus
}
#endif
