// Allocation-free routing counts.
//
// This entry point has no counterpart in the reference library.
//
// Who it is for: code that must not allocate device memory at the point where it needs the routing
// counts.  Typical cases are a caller that runs under a framework whose memory pool owns all device
// memory and forbids raw cudaMalloc/cudaFree (they synchronise the whole device and bypass the
// pool's accounting), a caller inside a latency-critical region where an implicit device
// synchronisation is not acceptable, and a plain C/C++ host that does not link PyTorch and so cannot
// use the tensor-allocating Python wrappers.  Such callers pass their own input and output buffers;
// the intermediate per-chunk histograms live in a fixed array inside the library.
//
// What it computes (same numbers as Buffer.get_dispatch_layout / route_hist): for topk_idx [T,K]
//   counts[0 .. E)          entries routed to each global expert
//   counts[E .. E+N)        tokens that reach each rank (a token counts once per rank)
//   counts[E+N]             sum over tokens of distinct destination ranks
//   counts[E+N+1]           T
// Entries outside [0, E) (for example -1) are ignored.
//
// Limits: T <= 65536 tokens, K <= 32, N <= 32 ranks, E + N + 2 <= 1088 columns.  Larger sizes are
// rejected with TMOE_NOALLOC_TOO_LARGE before anything is launched.  The scratch array
// (512 x 1088 ints = 2.2 MB) is part of the loaded library image: every GPU that loads the library
// holds it until the process exits.
//
// Behaviour to know about:
//  * The first call on a device looks up the device address of the scratch array
//    (cudaGetSymbolAddress) with that device current.  Make that first call outside any stream
//    capture; later calls only launch two kernels on `stream`.
//  * All calls share the one scratch array, and it keeps the previous call's contents.  Every call
//    overwrites the part it reads, so stale contents never leak into a result, but two calls whose
//    kernels overlap on the GPU (different streams, no dependency) race on it.  Serialise them.
//  * Nothing is allocated or freed: no cudaMalloc, cudaFree, or allocating library routine.
#pragma once
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    TMOE_NOALLOC_OK = 0,
    TMOE_NOALLOC_BAD_ARGUMENT = -1,  // null pointer, non-positive K/E/N, E not divisible by N
    TMOE_NOALLOC_TOO_LARGE = -2,     // a size exceeds the limits above
    TMOE_NOALLOC_CUDA_ERROR = -3,    // a CUDA call failed; the message holds cudaGetErrorString
};

// topk_idx: device pointer, [T,K] int64 (idx_is_64bit != 0) or int32.  counts_out: device pointer to
// E + N + 2 ints.  stream: a cudaStream_t (0 = default stream).  err / err_len: optional host buffer
// that receives a one-line message when the return value is not TMOE_NOALLOC_OK.
int tmoe_route_counts_noalloc(const void* topk_idx, int idx_is_64bit, int num_tokens, int top_k, int num_experts, int num_ranks,
                              int* counts_out, void* stream, char* err, size_t err_len);

#ifdef __cplusplus
}
#endif
