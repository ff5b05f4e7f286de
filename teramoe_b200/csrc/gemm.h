// Host interface of the hand-written tcgen05 grouped GEMM family (gemm.cu).
//
// All matrices are bf16, accumulation is fp32 in tensor memory.  "Slot space" is the per-rank
// expert-sorted row space in which every local expert owns a contiguous segment whose length is
// padded to a multiple of 128 rows; pad rows are zero and carry route weight 0.
//
// Reference counterparts: csrc/teramoe/teramoe_wrapper.cuh:530-780 (persistent UMMA GEMM),
// csrc/teramoe/teramoe_sm100_bf16_compute.cuh:567-746 (SwiGLU epilogue), the SIMT dSwiGLU loop at
// csrc/teramoe/teramoe_orchestrator.cu:4723-4784 (fused here into the GEMM epilogue) and the two
// QuACK weight-gradient GEMMs at teramoe/buffer.py:745-760 (replaced by gemm_wgrad).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tmoe {

// Destination of the "push" epilogues: output row s (a slot) is stored straight into the landing table
// of the rank that owns the token, at row slot_tk[s] (= t*K+k at the source), with peer stores over
// NVLink issued from the GEMM epilogue.  Pad rows (slot_tk < 0) are skipped.
struct PushTarget {
    const uint64_t* arena_ptrs = nullptr;  // device [ranks]: base address of every rank's symmetric arena
    uint64_t landing_off = 0;              // byte offset of the [T*K, H] landing table inside the arena
    const int* slot_tk = nullptr;          // device [slots]
    const int* slot_row = nullptr;         // device [slots]
    const int* recv_row_base = nullptr;    // device [ranks + 1]
    int num_ranks = 1;
};

// Returns cudaSuccess or the launch / tensor-map error.  `status` is a 4-int device block that the
// kernels fill when a bounded wait runs out (see ptx.cuh); may be nullptr.
//
// Block structure of slot space, shared by the M-grouped kernels.
struct MGroupLayout {
    const int* mblock_expert = nullptr;    // device [max_mblocks], local expert id of each 128-row block
    const int* num_mblocks_dev = nullptr;  // device scalar, number of live blocks (<= max_mblocks)
    int max_mblocks = 0;                   // rows allocated in slot space / 128
    // Optional: pairing of blocks for the CTA-pair (cta_group::2) kernels.  A unit is one or two
    // consecutive blocks of one expert; unit_blk[u] is its first block and unit_blk[num_units] the
    // block count.  When unit_blk is null the one-CTA kernels run.
    const int* unit_blk = nullptr;         // device [max_units + 1]
    const int* num_units_dev = nullptr;    // device scalar
    int max_units = 0;
};

// act[S,I] = silu(g) * u * row_w ; preact[S,2I] = (g,u) interleaved, with GU = xperm[S,H] . W_gateup[e]^T
// W_gateup is [E,2I,H] with rows element-interleaved (g0,u0,g1,u1,...).
cudaError_t gemm_fwd_gateup(const void* xperm, const void* w_gateup, void* act, void* preact, const float* row_w,
                            const MGroupLayout& lay, int H, int I, int num_local_experts, const int* gather_rows, int src_rows, int* status, int num_sms,
                            cudaStream_t stream);

// y[S,H] = act[S,I] . W_down[e]^T          (W_down [E,H,I])
// With `push` the rows are not written to y (may be null) but pushed to their source ranks (combine fused into
// the GEMM epilogue).
cudaError_t gemm_fwd_down(const void* act, const void* w_down, void* y, const MGroupLayout& lay, int H, int I,
                          int num_local_experts, int* status, int num_sms, cudaStream_t stream, const PushTarget* push = nullptr);

// ga = dy[S,H] . W_down[e]  (fp32, never stored), then fused dSwiGLU with the saved preact:
//   dgu[S,2I] interleaved (d_gate,d_up), act_w[S,I] = row_w * silu(g) * u (operand of dW_down),
//   droute_part[S, 2*ceil(I/256)] partial sums of ga * silu(g) * u (summed by reduce kernels).
cudaError_t gemm_bwd_gradact(const void* dyperm, const void* w_down, const void* preact, const float* row_w, void* dgu,
                             void* act_w, float* droute_part, const MGroupLayout& lay, int H, int I, int num_local_experts, const int* gather_rows, int src_rows,
                             int* status, int num_sms, cudaStream_t stream);

// dxperm[S,H] = dgu[S,2I] . W_gateup[e]
cudaError_t gemm_bwd_dx(const void* dgu, const void* w_gateup, void* dxperm, const MGroupLayout& lay, int H, int I,
                        int num_local_experts, int* status, int num_sms, cudaStream_t stream, const PushTarget* push = nullptr);

// dW[e] [M,N] = A[seg_e, M]^T . B[seg_e, N]  for every local expert, seg_e = rows
// [seg_offsets[e], seg_offsets[e+1]) of slot space (multiples of 128).  Empty segments give zeros.
//
// Gather modes (all kernels that take `gather_rows`): instead of a dense slot-space operand the kernel
// reads row gather_rows[s] of a row source [src_rows, cols] for slot row s (TMA tile::gather4; -1 reads
// zeros), so the token-once receive buffer feeds the GEMMs without an expanded copy.  For gemm_wgrad
// `gather_operand` says which operand is the row source: 1 = a, 2 = b, 0 = none.
cudaError_t gemm_wgrad(const void* a, const void* b, void* dw, const int* seg_offsets, int total_rows, int M, int N,
                       int num_local_experts, const int* gather_rows, int gather_operand, int src_rows, bool cta_pairs, int* status,
                       int num_sms, cudaStream_t stream);

int gemm_num_droute_parts(int I);

// Whether the TMA row-gather operand modes were compiled in (-DTMOE_WITH_GATHER4).
bool gemm_has_gather4();

}  // namespace tmoe
