// Host interface of the routing-preparation kernels (routing.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tmoe {

// Device arrays written by layout_finalize (E = global experts, N = ranks, El = E / N).
struct LayoutOut {
    int* expert_total;   // [E]   tokens routed to expert e from all ranks
    int* my_src_off;     // [E]   rows of lower source ranks inside expert e's segment
    int* seg_off_all;    // [E]   offset of expert e's padded segment inside its rank's slot space
    int* my_row_base;    // [N]   first row of this source's block in rank d's receive buffer
    int* recv_row_base;  // [N+1] this rank's receive buffer: first row of source s (last = total rows)
    int* seg_offsets;    // [El+1] this rank's padded segment offsets (rows of slot space)
    int* num_mblocks;    // [2]   live 128-row blocks of this rank; number of (token,k) entries this rank sends
    int* send_base;      // [E]   position of this rank's first entry for expert e in its send order
    int* sizes;          // [12]  rows, padded slots, landing rows of this rank; their maxima over ranks; blocks; max tokens;
                         //       [8] = 1 if the maxima fit the capacities given to layout_finalize (or none were given)
};

int route_chunk_tokens();

// in_rank (optional): [T, N] bytes, 1 where the token has an expert on that rank (is_token_in_rank of the layout API).
cudaError_t route_hist(const void* topk_idx, int is64, int T, int K, int E, int N, int* chunk_hist, uint8_t* in_rank, cudaStream_t stream);
// totals[c] = sum over chunks of chunk_hist[chunk][c]
cudaError_t route_sum(const int* chunk_hist, int num_chunks, int C, int* totals, cudaStream_t stream);
cudaError_t route_scan(const int* chunk_hist, int* chunk_base, int num_chunks, int E, int rank, int N, const uint64_t* meta_ptrs,
                       const uint64_t* signal_ptrs, int epoch, int* status, cudaStream_t stream);
// cap_*: capacities (rows, padded slots, tokens; maxima over ranks) of tables that were sized before the layout was known;
// cap_rows <= 0: no check.  The answer is out.sizes[8].
cudaError_t layout_finalize(const int* meta, int rank, int N, int E, const LayoutOut& out, int cap_rows, int cap_slots, int cap_tokens,
                            cudaStream_t stream);
cudaError_t slot_pad_fill(const int* seg_offsets, const int* expert_total_local, int e_local, int* slot_row, float* slot_w,
                          int* slot_tk, int* mblock_expert, int* unit_blk, int* num_units, const int* ok, cudaStream_t stream);
// send_order (optional, [T*K]): entries (t*K+k) of this rank in the order a fused dispatch sends them:
// destination ranks in rotation (own rank first, then rank+1, ...), experts ascending, ranks ascending.
cudaError_t route_assign(const void* topk_idx, int is64, int T, int K, int E, int N, const int* chunk_base, const LayoutOut& out,
                         int* send_slot, int* send_row, int* land_off, int* ndst, int* send_order, cudaStream_t stream);

// `ok` (here and in slot_pad_fill / arrival_order; may be null): device flag written by layout_finalize; 0 makes the kernel return.
cudaError_t zero_pad_rows(const int* seg_offsets, const int* expert_total_local, int e_local, void* slot_x, int H, const int* ok,
                          cudaStream_t stream);

// Arrival order for a fused dispatch + GEMM: blk_group[b] = latest arrival group (0..groups-1) among the
// sources of block b; unit_order = units of the CTA-pair GEMM sorted by arrival group (stable).
cudaError_t arrival_order(const int* meta, int rank, int N, int E, int groups, const int* seg_offsets, const int* unit_blk,
                          const int* num_units, int max_units, int* blk_group, int* unit_order, const int* ok, cudaStream_t stream);

}  // namespace tmoe
