// edgelm_attn_decode_noalloc: decode attention for callers that must not allocate.
//
// This entry point has no counterpart in adarsh-sgh/edgelm; it exists for users of this library.
//
// Who needs it: code that runs where device memory cannot be allocated: inside a region that
// another framework owns and has sized up front (a plugin called from someone else's runtime, a
// real-time loop that forbids allocator calls, a process whose memory pool is handed out once at
// start and then frozen).  The regular entry point, edgelm_attn_decode, asks its caller for two
// scratch buffers when the keys of a sequence are split over several blocks; such a caller has
// nowhere to get them from.  This variant keeps that scratch inside the library, in a
// file-scope device array, and takes inputs and outputs only.
//
// Limits and rules:
//  * The scratch holds EDGELM_NOALLOC_SCRATCH_FLOATS floats (4 MiB).  Every GPU that loads the
//    library holds that much memory until the process exits.  A call needs
//    n_seqs * n_heads * n_splits * (head_dim + 2) floats; a call that needs more is refused with
//    a message and launches nothing.  With n_splits == 1 no scratch is used.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress) and
//    remembers it for that device; with lazy module loading that call may also be the one that
//    loads the library's device code and so brings the array into being.  Make that first call
//    during set-up: before the region in which nothing may be allocated, and before any stream
//    capture.
//  * All calls share the one array, which keeps whatever the last call left in it.  Nothing in it
//    has to start at zero: every (sequence, head, split) cell that the second kernel reads has
//    been written by the first kernel of the same call.  Two calls that may run at the same time
//    on one GPU (different streams) race on the array: order them.
//  * It calls no cudaMalloc, cudaFree, or any routine that allocates.
//
// Arguments are those of edgelm_attn_decode without part_o and part_ml.  Returns 0, or a negative
// code with a message in edgelm_last_error().
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define EDGELM_NOALLOC_SCRATCH_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

int edgelm_attn_decode_noalloc(const void* q, int ldq, void* out, int ldo, const void* kcache, const void* vcache,
                               int dtype, const int32_t* page_table, int table_stride, const int32_t* seq_slot,
                               const int32_t* seq_pos, int n_seqs, int nh, int nkv, int hd, float scale, int n_splits,
                               cudaStream_t stream);

#ifdef __cplusplus
}
#endif
