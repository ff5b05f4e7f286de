// Host interface of the low-latency (inference-style) dispatch / combine kernels (lowlat.cu).
//
// One NVSwitch node, push to final place: a sender stores every message straight into the window
// [local expert][source rank][slot] of the destination rank and then publishes the window's row count with ONE
// 8-byte release store; the receiver waits (bounded) for the counts, packs the windows of an expert back to back and
// records where every source's rows went.  Combine sends expert outputs back to [global expert][token] windows of
// the token's rank, which forms the weighted sum.  Flags carry the call number, so nothing has to be cleaned between
// calls and no double buffering is needed.
//
// Reference counterparts: csrc/kernels/internode_ll.cu:129-463 (dispatch: per-128-channel FP8 cast in flight, push
// to the per-expert slot, arrival flag, per-source wait statistics, time-out -> mask), :557-713 (LogFMT-10),
// :715-1139 (weighted combine), :1241-1288 (mask kernels), csrc/config.hpp:133-219 (buffer layout).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tmoe {

// Byte geometry of the low-latency windows inside every rank's symmetric arena (same on all ranks).
struct LowLatLayout {
    int num_ranks, rank, num_experts, max_tokens, hidden;
    int use_fp8;              // dispatch payload: e4m3 + one scale per 128 channels (else bf16)
    int use_ue8m0;            // scales as power-of-two exponents, four per 32-bit word
    int round_scale;          // scales rounded up to a power of two
    int use_logfmt;           // combine payload: LogFMT-10 per 128 channels where it applies (else bf16)
    uint64_t off_d_stage;     // [E_local][ranks][max_tokens] messages of d_msg_bytes
    uint64_t off_d_flags;     // [E_local][ranks] int64: call number << 32 | rows + 1
    uint64_t off_c_stage;     // [experts][max_tokens] rows of c_row_bytes
    uint64_t off_c_flags;     // [experts] int64: call number << 32 | 1
    uint32_t d_msg_bytes;     // 16-byte header (source token) + payload + scales, multiple of 16
    uint32_t c_row_bytes;     // bf16: 2*hidden; LogFMT: hidden/128 groups of kLogfmtGroupBytes
};

constexpr int kLogfmtGroupBytes = 272;   // 4-byte header (bf16 amax, bf16 amin; amax bits 0 = the group is plain bf16) + up to 256 bytes

// mask: optional int[ranks] on the device (1 = the rank is ignored: nothing is sent to it, nothing is awaited from it).
// shrink != 0: a wait that runs out sets mask[rank] instead of reporting an error (elastic shrink).
// wait_stats: optional int64[ranks], nanoseconds spent waiting for each source are added.
cudaError_t ll_dispatch_send(const LowLatLayout& lay, const void* x, const void* topk_idx, int idx_is64, int T, int K,
                             const uint64_t* arena_ptrs, long long call_seq, const int* mask, cudaStream_t stream);

// recv_x: [E_local, ranks*max_tokens, hidden] e4m3 or bf16; recv_scales: fp32 [E_local, hidden/128, ranks*max_tokens] or
// int32 [E_local, hidden/512, ranks*max_tokens] (UE8M0), i.e. column-major per expert; src_info [E_local, ranks*max_tokens];
// layout_range int64 [E_local, ranks] = count << 32 | begin; recv_count [E_local]; expert_stats optional int [E_local] (+=).
cudaError_t ll_dispatch_recv(const LowLatLayout& lay, const void* arena_local, void* recv_x, void* recv_scales, int* src_info,
                             long long* layout_range, int* recv_count, int* expert_stats, long long* wait_stats, long long call_seq,
                             int* mask, int shrink, uint64_t limit_ns, int* status, cudaStream_t stream);

// x: [E_local, ranks*max_tokens, hidden] bf16 expert outputs in the packed layout of the dispatch.
cudaError_t ll_combine_send(const LowLatLayout& lay, const void* x, const int* src_info, const long long* layout_range,
                            const uint64_t* arena_ptrs, long long call_seq, const int* mask, cudaStream_t stream);

// out[t] = sum_k topk_weights[t,k] * row of (expert topk_idx[t,k], token t); rows of masked ranks count as zero.
cudaError_t ll_combine_recv(const LowLatLayout& lay, const void* arena_local, const void* topk_idx, int idx_is64, const float* topk_weights,
                            int T, int K, void* out, long long* wait_stats, long long call_seq, int* mask, int shrink, uint64_t limit_ns,
                            int* status, cudaStream_t stream);

// Rank-mask maintenance (reference: query / update / clean mask buffer kernels).
cudaError_t ll_mask_update(int* mask, int num_ranks, int rank, int value, cudaStream_t stream);
cudaError_t ll_mask_query(const int* mask, int num_ranks, int* out, cudaStream_t stream);
cudaError_t ll_mask_clean(int* mask, int num_ranks, cudaStream_t stream);

}  // namespace tmoe
