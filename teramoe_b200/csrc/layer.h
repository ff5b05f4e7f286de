// Host interface of the whole-layer kernel (layer.cu): ONE cooperative persistent launch per direction that runs
// dispatch, both grouped GEMMs with their fused epilogues, the combine push, the weight gradients (backward) and the
// reduce of the landed rows, driven by a work list that a small scheduler kernel builds on the device.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "fused.h"
#include "gemm.h"

namespace tmoe {

// Kinds of work-list items.  An item is an int4 that carries its whole geometry:
//   x  bits 0-3 kind, bit 4 "the unit has two blocks", bits 8-27 local expert
//   first / second GEMM:  y = unit, z = column block | rows awaited in block 0 << 16 | rows awaited in block 1 << 24, w = first block
//   weight gradients:     y = first slot row of the expert, z = column block | row unit of dW << 16, w = number of 64-row K blocks
enum LayerWorkKind : int {
    kWorkGemm1 = 0,        // forward: gate_up + SwiGLU    backward: grad_act + dSwiGLU
    kWorkGemm2 = 1,        // forward: down + push         backward: dX + push (+ route gradients)
    kWorkWgradDown = 2,    // backward only
    kWorkWgradGateup = 3,  // backward only
    kWorkReduce = 4,       // not an item: the gather role (own token counter); the number names its time stamps
};

// Optional time counters of one launch (nanoseconds, summed over the threads that waited; divide by the number of CTA
// pairs for a per-pair mean).  The reference has no counterpart in its fused kernel (only the low-latency kernels
// record wait cycles per source rank, csrc/kernels/internode_ll.cu:385-418).
enum LayerStat : int {
    kStatWaitArrival = 0,    // producers waiting for dispatched rows of other ranks (first GEMM)
    kStatWaitFirstGemm = 1,  // producers waiting for a unit's first GEMM (second GEMM)
    kStatWaitWgrad = 2,      // producers checking / waiting for an expert's units (weight gradients)
    kStatWaitLanded = 3,     // gather: waiting for every rank's "pushes complete" (one thread per CTA)
    kStatKindFirst = 8,      // + kind: ~(globaltimer) when the first item of that kind was taken by an epilogue (max of the complement)
    kStatKindLast = 16,      // + kind: globaltimer when the last item of that kind was finished by an epilogue
    kLayerStatWords = 24,
};

struct LayerParams {
    int bwd;                       // 0 forward, 1 backward
    int H, I, El, slot_rows;       // slot_rows: rows of the slot-space operand table in the arena (multiple of 128)
    int out_rows;                  // rows of out0 / out1 / preact / droute_part / xperm (multiple of 128, >= this rank's padded slots)
    int T, K, E, N, rank;
    const void* slot_x;            // [slot_rows, H] operand table inside this rank's arena (peers fill it)
    const void* w1;                // forward W_gateup [El,2I,H]   backward W_down [El,H,I]
    const void* w2;                // forward W_down [El,H,I]      backward W_gateup [El,2I,H]
    void* out0;                    // forward act [out_rows, I]       backward act x route [out_rows, I]
    void* out1;                    // forward preact [out_rows, 2I]   backward dGU [out_rows, 2I]
    const void* preact;            // backward: saved pre-activation
    float* droute_part;            // backward: [out_rows, 2*ceil(I/256)] route-gradient partial sums
    const float* row_w;            // route weight per slot row
    const void* xperm;             // backward: X in slot space [out_rows, H] (operand of dW_gateup)
    const void* x_rows;            // backward, optional: [rows, H] X once per received token; then the kernel fills xperm itself
    int expand_rows;               //   (rows 0 .. expand_rows-1, through push.slot_row) while the first GEMMs run
    void* dw_down;                 // backward: [El, H, I]
    void* dw_gateup;               // backward: [El, 2I, H]
    MGroupLayout lay;
    const int* seg_offsets;        // [El + 1]
    const int* expert_total_local; // [El]
    const int* unit_order;         // [max_units] units in arrival order
    // work list and counters (device memory of the caller; `sync` must be zero before the launch)
    void* work;                    // int4 [max_work]
    int max_work;
    int* num_work;                 // device scalar written by the scheduler kernel
    int* expert_units;             // int2 [El]: first unit and unit count of every local expert (written by the scheduler)
    int* sync;                     // [8 + max_units]: item counter, finished-push counter, complete units, gather token counter, X rows claimed / filled, next unit of the replicate role, 1 spare,
                                   //   finished first-GEMM warps per unit
    int group_units;               // units per batch of the schedule (compute_batch_size / 256)
    int lag_percent;               // how far (percent of a batch) the first GEMM runs ahead before the batch's second GEMM starts
    int min_lag_items;             // lower bound of that distance in first-GEMM items (0: none); about two per CTA pair avoids waiting
    int reduce_chunk;              // tokens per reduce item
    PushTarget push;
    uint64_t gtw_off;              // backward: byte offset of the route-gradient table in the arenas
    const uint64_t* signal_ptrs;   // [N] every rank's signal row (int[N]) in the control arena
    const int* my_signal;          // this rank's signal row
    int epoch;                     // value that says "my pushes of this call are complete"
    const void* landing;           // [T*K, H] this rank's landing table
    void* out;                     // [T, H]
    const float* gtw_in;           // backward: [T*K] route gradients that arrived
    float* gtw_out;                // backward: [T, K]
    FusedArgs f;                   // dispatch role
    unsigned long long* stats;     // optional [kLayerStatWords], zero before the launch
    const int* geom_ok;            // optional device flag (layout_finalize): 0 = the layout does not fit the tables, do nothing
    int* status;
    int num_sms;
};

// Upper bound on work items for the given shapes (host side, for sizing `work`).
int moe_layer_max_work(int bwd, int max_units, int H, int I, int El, int T, int reduce_chunk);

// The scheduler kernel alone (moe_layer_launch runs it first): needs bwd, H, I, El, T, lay.num_units_dev / max_units,
// lay.unit_blk / mblock_expert, unit_order, seg_offsets, expert_total_local, the schedule knobs and the work tensors of `p`.
cudaError_t moe_layer_schedule(const LayerParams& p, cudaStream_t stream);

cudaError_t moe_layer_launch(const LayerParams& p, cudaStream_t stream);

}  // namespace tmoe
