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
    int* num_mblocks;    // [1]
    int* sizes;          // [8]   rows, padded slots, landing rows of this rank; their maxima over ranks; blocks; max tokens
};

int route_chunk_tokens();

cudaError_t route_hist(const void* topk_idx, int is64, int T, int K, int E, int N, int* chunk_hist, cudaStream_t stream);
cudaError_t route_scan(const int* chunk_hist, int* chunk_base, int num_chunks, int E, int rank, int N, const uint64_t* meta_ptrs,
                       const uint64_t* signal_ptrs, int epoch, int* status, cudaStream_t stream);
cudaError_t layout_finalize(const int* meta, int rank, int N, int E, const LayoutOut& out, cudaStream_t stream);
cudaError_t slot_pad_fill(const int* seg_offsets, const int* expert_total_local, int e_local, int* slot_row, float* slot_w,
                          int* slot_tk, int* mblock_expert, int* unit_blk, int* num_units, cudaStream_t stream);
cudaError_t route_assign(const void* topk_idx, int is64, int T, int K, int E, int N, const int* chunk_base, const LayoutOut& out,
                         int* send_slot, int* send_row, int* land_off, int* ndst, cudaStream_t stream);

}  // namespace tmoe
