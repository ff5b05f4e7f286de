// Host interface of the expert-parallel data-movement kernels (comm.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tmoe {

// Byte offsets of the peer-visible tables inside every rank's symmetric arena (same on all ranks).
struct SymOffsets {
    uint64_t recv_x;     // [row_cap, H] bf16   token rows, once per (source token, this rank)
    uint64_t slot_row;   // [slot_cap] int      receive row feeding each slot (-1 = pad)
    uint64_t slot_w;     // [slot_cap] float    route weight of the slot (0 = pad)
    uint64_t slot_tk;    // [slot_cap] int      t*K+k of the entry at its source (-1 = pad)
    uint64_t row_tok;    // [row_cap] int       token index at the source
    uint64_t row_land;   // [row_cap] int       landing row at the source
    uint64_t row_slots;  // [row_cap, K] int    slots of the row's local expert hits (-1 padded)
    uint64_t landing;    // [land_cap, H] bf16  combine landing rows (one per token and destination rank)
    uint64_t gtw;        // [tok_cap*K] float   route-weight gradients arriving from expert ranks
    uint64_t row_topk_idx;  // [row_cap, K] int64  LOCAL expert id of each of the row's top-k entries, -1 for experts of other ranks
    uint64_t row_topk_w;    // [row_cap, K] float  route weight of those entries, 0 elsewhere
};

// limit_ms <= 0 selects the run-time limit of the status block (ptx.cuh).
// mode 0: barrier (signal every rank, wait for every rank); 1: signal only (never waits); 2: wait only.
// The signal-only / wait-only forms on a second flag row are the release / acquire of the data arena between calls.
// mask (optional, int[N] on the device): ranks with a non-zero entry are neither signalled nor waited for.
cudaError_t ep_barrier(const uint64_t* signal_ptrs, int rank, int N, int epoch, int* status, int site, int limit_ms, int mode,
                       const int* mask, cudaStream_t stream);

cudaError_t dispatch_push(const void* x, const void* topk_idx, int is64, const float* topk_w, int T, int K, int H, int E, int N,
                          const int* send_slot, const int* send_row, const int* land_off, const uint64_t* arena_ptrs,
                          const SymOffsets& so, int with_meta, int num_blocks, const int* ok /* optional device flag, 0: send nothing */,
                          cudaStream_t stream);

// Rows [*rows_dev, total_rows) of fixed-shape dispatch outputs become "nothing": zero payload, expert id -1, weight 0.
cudaError_t tail_fill(void* x, int64_t* idx, float* w, const int* rows_dev, int total_rows, int H, int K, cudaStream_t stream);

cudaError_t expand_rows(const void* rows, const int* slot_row, void* out, int num_slots, int H, cudaStream_t stream);

cudaError_t combine_push(const void* y, const int* row_slots, const int* row_land, const int* recv_row_base, int R, int K, int H,
                         int N, const uint64_t* arena_ptrs, const SymOffsets& so, const float* droute_part, int n_parts,
                         const int* slot_tk, int with_payload, int num_blocks, cudaStream_t stream);

cudaError_t combine_reduce(const void* landing, const int* land_off, const int* ndst, void* out, int T, int H, cudaStream_t stream);

// Fused-combine path: the down / dX GEMM epilogues store one row per (token,k) entry into the landing
// table [T*K, H] of the token's rank; the reduce sums a token's valid entries.
cudaError_t combine_reduce_slots(const void* landing, const void* topk_idx, int is64, void* out, int T, int K, int H, int E,
                                 const float* weights /* optional [T,K] */, cudaStream_t stream);
cudaError_t slot_rows_push(const void* y, const int* slot_tk, const int* slot_row, const int* recv_row_base, int S, int H, int N,
                           const uint64_t* arena_ptrs, uint64_t landing_off, cudaStream_t stream);
cudaError_t droute_push(const float* droute_part, int n_parts, const int* slot_tk, const int* slot_row, const int* recv_row_base, int S,
                        int N, const uint64_t* arena_ptrs, uint64_t gtw_off, cudaStream_t stream);

cudaError_t numerics_check(const void* a, const void* b, long n, int is_bf16, double* out6, cudaStream_t stream);

}  // namespace tmoe
