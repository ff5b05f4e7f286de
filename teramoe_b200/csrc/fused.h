// Host interface of the fused dispatch + grouped GEMM kernel (fused.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm.h"

namespace tmoe {

// What the dispatch pairs need.  Offsets are byte offsets inside every rank's symmetric data arena
// (arena_ptrs) or control arena (ctrl_ptrs); they are the same on all ranks.
struct FusedArgs {
    int num_dispatch_clusters;     // CTA pairs that dispatch first and then join the others on the GEMM tiles
    int* tile_counter;             // device int, zero before the kernel: next GEMM tile to claim
    const void* x;                 // [T, H] bf16 rows to send (x in forward, grad_out in backward)
    const void* topk_idx;          // [T, K]
    int idx_is64;
    const float* topk_w;           // [T, K] (forward)
    const int* send_order;         // [max_send] entries t*K+k in sending order
    const int* num_send;           // device scalar
    int max_send;
    const int* send_slot;          // [T*K] slot on the destination rank
    const int* send_row;           // [T, N] receive row on the destination rank
    int T, K, H, E, N;
    int with_meta;                 // forward: also store the slot tables
    int slot_cap;                  // rows of the destination operand table
    const uint64_t* arena_ptrs;    // [N]
    const uint64_t* ctrl_ptrs;     // [N]
    uint64_t off_slot_x, off_slot_w, off_slot_tk, off_slot_row, off_row_first;   // in the data arena
    uint64_t off_blk_cnt;          // in the control arena: int per 128-row block, zero before the kernel
    // what the compute pairs need beyond the GEMM arguments
    const int* blk_cnt;            // this rank's arrival counters (local view of off_blk_cnt)
    const int* unit_order;         // units sorted by arrival group
    const int* seg_offsets;        // [El + 1]
    const int* expert_total_local; // [El]
    // Whole-layer kernel only: one row per (token, destination rank) on the wire.  The entries of a token on one rank
    // share the row that travels to the entry with the smallest slot there (its "home"); the others only get their
    // table entries and `slot_src` = the home slot, and the receiver copies the row locally (gather warps) before it
    // counts the block as ready.  0: one row per (token, k) entry, every slot is filled by its sender.
    int wire_rank;
    uint64_t off_slot_src;         // data arena: int per slot; -1 = the row itself arrives, else the slot to copy it from
    const int* slot_src;           // this rank's view of that table
    int* blk_ready;                // local, zero before the kernel: rows in place (arrived or copied) per 128-row block
    int* replicate_counter;        // local, zero before the kernel: next unit (in arrival order) whose blocks get their copies
};

struct GemmArgsPublic {
    MGroupLayout lay;
    int H, I, num_local_experts;
    const float* row_w;            // slot route weights (forward: the table the dispatchers fill)
    void* out0;                    // forward: act [S, I]      backward: act_w [S, I]
    void* out1;                    // forward: preact [S, 2I]  backward: dGU [S, 2I]
    const void* preact;            // backward input
    float* droute_part;            // backward: [S, 2*ceil(I/256)]
    int* status;
};

// kind 0: forward (rows = X, weights = W_gateup [E,2I,H]); kind 1: backward (rows = dY, weights = W_down [E,H,I]).
// slot_x is this rank's operand table inside the arena ([slot_rows, H], slot_rows a multiple of 128).
cudaError_t fused_dispatch_gemm(int kind, const void* slot_x, int slot_rows, const void* w, const GemmArgsPublic& p, const FusedArgs& f,
                                int num_sms, cudaStream_t stream);

}  // namespace tmoe
