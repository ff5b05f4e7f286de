// Bindings for routing preparation, expert-parallel data movement and the symmetric-memory runtime.
// Kernels take torch tensors; tables that live in the symmetric arena are passed as tensor views
// created by SymmetricArena.view (no copy, no ownership).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "comm.h"
#include "fused.h"
#include "launch_count.h"
#include "layer.h"
#include "lowlat.h"
#include "routing.h"
#include "runtime.h"

namespace {

#define TM_CHECK_CUDA(call)                                                                          \
    do {                                                                                             \
        tmoe::count_launch();                                                                        \
        cudaError_t _e = (call);                                                                     \
        TORCH_CHECK(_e == cudaSuccess, "teramoe_b200: ", #call, " failed: ", cudaGetErrorString(_e)); \
    } while (0)

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

int* i32(const torch::Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kInt32 && t.is_contiguous(), name, " must be a contiguous int32 CUDA tensor");
    return t.data_ptr<int>();
}
float* f32(const torch::Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kFloat32 && t.is_contiguous(), name, " must be a contiguous fp32 CUDA tensor");
    return t.data_ptr<float>();
}
const uint64_t* u64(const torch::Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kInt64 && t.is_contiguous(), name, " must be a contiguous int64 CUDA tensor");
    return reinterpret_cast<const uint64_t*>(t.data_ptr<int64_t>());
}
void* bf16(const torch::Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kBFloat16 && t.is_contiguous(), name, " must be a contiguous bf16 CUDA tensor");
    return t.data_ptr();
}
void check_i32(const torch::Tensor& t, const char* name) { (void)i32(t, name); }
int* opt_status(const c10::optional<torch::Tensor>& s) {
    if (!s.has_value()) return nullptr;
    TORCH_CHECK(s->numel() >= 8, "status must hold 8 ints");
    return i32(*s, "status");
}

struct TopK {
    const void* ptr;
    int is64, T, K;
};
TopK topk(const torch::Tensor& idx) {
    TORCH_CHECK(idx.is_cuda() && idx.is_contiguous() && idx.dim() == 2, "topk_idx must be a contiguous [T,K] CUDA tensor");
    TORCH_CHECK(idx.scalar_type() == torch::kInt64 || idx.scalar_type() == torch::kInt32, "topk_idx must be int64 or int32");
    return TopK{idx.data_ptr(), idx.scalar_type() == torch::kInt64 ? 1 : 0, (int)idx.size(0), (int)idx.size(1)};
}

tmoe::LayoutOut layout_out(const std::vector<torch::Tensor>& t) {
    TORCH_CHECK(t.size() == 9, "layout tensor list must have 9 entries");
    tmoe::LayoutOut o;
    o.expert_total = i32(t[0], "expert_total");
    o.my_src_off = i32(t[1], "my_src_off");
    o.seg_off_all = i32(t[2], "seg_off_all");
    o.my_row_base = i32(t[3], "my_row_base");
    o.recv_row_base = i32(t[4], "recv_row_base");
    o.seg_offsets = i32(t[5], "seg_offsets");
    o.num_mblocks = i32(t[6], "num_mblocks");
    o.sizes = i32(t[7], "sizes");
    o.send_base = i32(t[8], "send_base");
    TORCH_CHECK(t[6].numel() >= 2, "num_mblocks must hold 2 ints");
    TORCH_CHECK(t[7].numel() >= 12, "sizes must hold 12 ints");
    return o;
}

tmoe::SymOffsets sym_offsets(const std::vector<int64_t>& v) {
    TORCH_CHECK(v.size() == 11, "need 11 symmetric offsets");
    tmoe::SymOffsets so;
    so.recv_x = v[0]; so.slot_row = v[1]; so.slot_w = v[2]; so.slot_tk = v[3]; so.row_tok = v[4];
    so.row_land = v[5]; so.row_slots = v[6]; so.landing = v[7]; so.gtw = v[8]; so.row_topk_idx = v[9]; so.row_topk_w = v[10];
    return so;
}

void route_hist(torch::Tensor topk_idx, int64_t E, int64_t N, torch::Tensor chunk_hist, c10::optional<torch::Tensor> in_rank) {
    const TopK tk = topk(topk_idx);
    uint8_t* ir = nullptr;
    if (in_rank.has_value()) {
        TORCH_CHECK(in_rank->is_cuda() && in_rank->scalar_type() == torch::kBool && in_rank->is_contiguous() &&
                    in_rank->numel() == (int64_t)tk.T * N, "in_rank must be a contiguous bool [T, N] CUDA tensor");
        ir = reinterpret_cast<uint8_t*>(in_rank->data_ptr<bool>());
    }
    c10::cuda::CUDAGuard guard(topk_idx.device());
    TM_CHECK_CUDA(tmoe::route_hist(tk.ptr, tk.is64, tk.T, tk.K, (int)E, (int)N, i32(chunk_hist, "chunk_hist"), ir, cur_stream()));
}

void route_sum(torch::Tensor chunk_hist, int64_t num_chunks, int64_t C, torch::Tensor totals) {
    TORCH_CHECK(chunk_hist.numel() >= num_chunks * C && totals.numel() >= C, "route_sum: sizes");
    c10::cuda::CUDAGuard guard(chunk_hist.device());
    TM_CHECK_CUDA(tmoe::route_sum(i32(chunk_hist, "chunk_hist"), (int)num_chunks, (int)C, i32(totals, "totals"), cur_stream()));
}

void route_scan(torch::Tensor chunk_hist, torch::Tensor chunk_base, int64_t num_chunks, int64_t E, int64_t rank, int64_t N,
                torch::Tensor meta_ptrs, torch::Tensor signal_ptrs, int64_t epoch, c10::optional<torch::Tensor> status) {
    c10::cuda::CUDAGuard guard(chunk_hist.device());
    TM_CHECK_CUDA(tmoe::route_scan(i32(chunk_hist, "chunk_hist"), i32(chunk_base, "chunk_base"), (int)num_chunks, (int)E, (int)rank, (int)N,
                                   u64(meta_ptrs, "meta_ptrs"), u64(signal_ptrs, "signal_ptrs"), (int)epoch, opt_status(status),
                                   cur_stream()));
}

void layout_finalize(torch::Tensor meta, int64_t rank, int64_t N, int64_t E, std::vector<torch::Tensor> layout, int64_t cap_rows,
                     int64_t cap_slots, int64_t cap_tokens) {
    c10::cuda::CUDAGuard guard(meta.device());
    TM_CHECK_CUDA(tmoe::layout_finalize(i32(meta, "meta"), (int)rank, (int)N, (int)E, layout_out(layout), (int)cap_rows, (int)cap_slots,
                                        (int)cap_tokens, cur_stream()));
}

void slot_pad_fill(torch::Tensor seg_offsets, torch::Tensor expert_total_local, torch::Tensor slot_row, torch::Tensor slot_w,
                   torch::Tensor slot_tk, torch::Tensor mblock_expert, c10::optional<torch::Tensor> unit_blk,
                   c10::optional<torch::Tensor> num_units, c10::optional<torch::Tensor> ok) {
    c10::cuda::CUDAGuard guard(seg_offsets.device());
    TM_CHECK_CUDA(tmoe::slot_pad_fill(i32(seg_offsets, "seg_offsets"), i32(expert_total_local, "expert_total_local"),
                                      (int)expert_total_local.numel(), i32(slot_row, "slot_row"), f32(slot_w, "slot_w"),
                                      i32(slot_tk, "slot_tk"), i32(mblock_expert, "mblock_expert"),
                                      unit_blk.has_value() ? i32(*unit_blk, "unit_blk") : nullptr,
                                      num_units.has_value() ? i32(*num_units, "num_units") : nullptr,
                                      ok.has_value() ? i32(*ok, "ok") : nullptr, cur_stream()));
}

void route_assign(torch::Tensor topk_idx, int64_t E, int64_t N, torch::Tensor chunk_base, std::vector<torch::Tensor> layout,
                  torch::Tensor send_slot, torch::Tensor send_row, torch::Tensor land_off, torch::Tensor ndst,
                  c10::optional<torch::Tensor> send_order) {
    const TopK tk = topk(topk_idx);
    c10::cuda::CUDAGuard guard(topk_idx.device());
    TM_CHECK_CUDA(tmoe::route_assign(tk.ptr, tk.is64, tk.T, tk.K, (int)E, (int)N, i32(chunk_base, "chunk_base"), layout_out(layout),
                                     i32(send_slot, "send_slot"), i32(send_row, "send_row"), i32(land_off, "land_off"),
                                     i32(ndst, "ndst"), send_order.has_value() ? i32(*send_order, "send_order") : nullptr, cur_stream()));
}

void arrival_order(torch::Tensor meta, int64_t rank, int64_t N, int64_t E, int64_t groups, torch::Tensor seg_offsets, torch::Tensor unit_blk,
                   torch::Tensor num_units, torch::Tensor blk_group, torch::Tensor unit_order, c10::optional<torch::Tensor> ok) {
    c10::cuda::CUDAGuard guard(meta.device());
    TM_CHECK_CUDA(tmoe::arrival_order(i32(meta, "meta"), (int)rank, (int)N, (int)E, (int)groups, i32(seg_offsets, "seg_offsets"),
                                      i32(unit_blk, "unit_blk"), i32(num_units, "num_units"), (int)unit_blk.numel() - 1,
                                      i32(blk_group, "blk_group"), i32(unit_order, "unit_order"), ok.has_value() ? i32(*ok, "ok") : nullptr,
                                      cur_stream()));
}

void zero_pad_rows(torch::Tensor seg_offsets, torch::Tensor expert_total_local, torch::Tensor slot_x, c10::optional<torch::Tensor> ok) {
    c10::cuda::CUDAGuard guard(slot_x.device());
    TM_CHECK_CUDA(tmoe::zero_pad_rows(i32(seg_offsets, "seg_offsets"), i32(expert_total_local, "expert_total_local"),
                                      (int)expert_total_local.numel(), bf16(slot_x, "slot_x"), (int)slot_x.size(1),
                                      ok.has_value() ? i32(*ok, "ok") : nullptr, cur_stream()));
}

// Fused dispatch + GEMM.  kind 0 forward (gate_up + SwiGLU), 1 backward (grad_act + dSwiGLU).
//   gemm_t : [slot_x view, weights, row_w, out0, out1] (+ [preact, droute_part] for kind 1)
//   layout : [mblock_expert, num_mblocks, unit_blk, num_units]
//   send_t : [x, topk_idx, send_order, num_send, send_slot, send_row] (+ [topk_w] when with_meta)
//   sym_t  : [arena_ptrs, ctrl_ptrs, blk_cnt view, unit_order, seg_offsets, expert_total_local, tile_counter (int, zero)]
//   offs   : [slot_x, slot_w, slot_tk, slot_row, row_first, blk_cnt(control arena)]
void fused_dispatch_gemm(int64_t kind, std::vector<torch::Tensor> gemm_t, std::vector<torch::Tensor> layout,
                         std::vector<torch::Tensor> send_t, std::vector<torch::Tensor> sym_t, std::vector<int64_t> offs, int64_t E,
                         int64_t N, bool with_meta, int64_t num_dispatch_clusters, c10::optional<torch::Tensor> status, int64_t num_sms) {
    TORCH_CHECK(gemm_t.size() == (kind == 0 ? 5u : 7u) && layout.size() == 4 && send_t.size() == (with_meta ? 7u : 6u) &&
                sym_t.size() == 7 && offs.size() == 6, "fused_dispatch_gemm: wrong argument lists");
    const torch::Tensor& slot_x = gemm_t[0];
    const torch::Tensor& w = gemm_t[1];
    const int S = (int)slot_x.size(0), H = (int)slot_x.size(1);
    tmoe::GemmArgsPublic p{};
    check_i32(layout[0], "mblock_expert");
    p.lay.mblock_expert = layout[0].data_ptr<int>();
    p.lay.num_mblocks_dev = i32(layout[1], "num_mblocks");
    p.lay.max_mblocks = S / 128;
    p.lay.unit_blk = i32(layout[2], "unit_blk");
    p.lay.num_units_dev = i32(layout[3], "num_units");
    p.lay.max_units = (int)layout[2].numel() - 1;
    p.H = H;
    p.num_local_experts = (int)w.size(0);
    p.I = kind == 0 ? (int)w.size(1) / 2 : (int)w.size(2);
    p.row_w = f32(gemm_t[2], "row_w");
    p.out0 = bf16(gemm_t[3], "out0");
    p.out1 = bf16(gemm_t[4], "out1");
    if (kind == 1) {
        p.preact = bf16(gemm_t[5], "preact");
        p.droute_part = f32(gemm_t[6], "droute_part");
    }
    p.status = opt_status(status);
    const TopK tk = topk(send_t[1]);
    tmoe::FusedArgs f{};
    f.num_dispatch_clusters = (int)num_dispatch_clusters;
    f.x = bf16(send_t[0], "x");
    f.topk_idx = tk.ptr;
    f.idx_is64 = tk.is64;
    f.send_order = i32(send_t[2], "send_order");
    f.num_send = i32(send_t[3], "num_send");
    f.max_send = (int)send_t[2].numel();
    f.send_slot = i32(send_t[4], "send_slot");
    f.send_row = i32(send_t[5], "send_row");
    f.topk_w = with_meta ? f32(send_t[6], "topk_w") : nullptr;
    f.T = tk.T; f.K = tk.K; f.H = H; f.E = (int)E; f.N = (int)N;
    f.with_meta = with_meta ? 1 : 0;
    f.slot_cap = S;
    f.arena_ptrs = u64(sym_t[0], "arena_ptrs");
    f.ctrl_ptrs = u64(sym_t[1], "ctrl_ptrs");
    f.blk_cnt = i32(sym_t[2], "blk_cnt");
    f.unit_order = i32(sym_t[3], "unit_order");
    f.seg_offsets = i32(sym_t[4], "seg_offsets");
    f.expert_total_local = i32(sym_t[5], "expert_total_local");
    check_i32(sym_t[6], "tile_counter");
    f.tile_counter = sym_t[6].data_ptr<int>();
    f.off_slot_x = offs[0]; f.off_slot_w = offs[1]; f.off_slot_tk = offs[2]; f.off_slot_row = offs[3]; f.off_row_first = offs[4];
    f.off_blk_cnt = offs[5];
    TORCH_CHECK(send_t[0].size(1) == H && S % 128 == 0 && sym_t[2].numel() >= S / 128, "fused_dispatch_gemm: shape mismatch");
    c10::cuda::CUDAGuard guard(slot_x.device());
    TM_CHECK_CUDA(tmoe::fused_dispatch_gemm((int)kind, bf16(slot_x, "slot_x"), S, bf16(w, "weights"), p, f, (int)num_sms, cur_stream()));
}

// Whole-layer kernel (layer.cu).
//   gemm_t : forward  [slot_x view, W_gateup, W_down, act, preact, row_w]
//            backward [slot_x view, W_down, W_gateup, act_w, dGU, row_w, preact, droute_part, xperm, dW_down, dW_gateup]
//   layout : [mblock_expert, num_mblocks, unit_blk, num_units, seg_offsets, expert_total_local, unit_order]
//   send_t : [x, topk_idx, send_order, num_send, send_slot, send_row] (+ [topk_w] in forward)
//   sym_t  : [arena_ptrs, ctrl_ptrs, blk_cnt view, signal_ptrs, my_signal view]
//   offs   : [slot_x, slot_w, slot_tk, slot_row, row_first, blk_cnt (control arena), landing, gtw]
//   push_t : [slot_tk, slot_row, recv_row_base]
//   red_t  : [landing view, out] (+ [gtw view, gtw_out] in backward)
//   work_t : [work (int32, 4 per item), num_work, expert_units (int32, 2 per expert), sync (zeroed, 8 + max_units)]
//   wire_t : [] = one row per (token, k) entry on the wire; [slot_src view (arena), blk_ready (zeroed, one int per 128-row
//            block)] = one row per (token, rank), copied into the token's other slots on the receiver; offs then has a ninth
//            entry, the byte offset of slot_src in the arenas
void moe_layer(bool bwd, std::vector<torch::Tensor> gemm_t, std::vector<torch::Tensor> layout, std::vector<torch::Tensor> send_t,
               std::vector<torch::Tensor> sym_t, std::vector<int64_t> offs, std::vector<torch::Tensor> push_t,
               std::vector<torch::Tensor> red_t, std::vector<torch::Tensor> work_t, int64_t E, int64_t N, int64_t rank, int64_t epoch,
               int64_t num_dispatch_clusters, int64_t group_units, int64_t lag_percent, int64_t min_lag_items, int64_t reduce_chunk,
               c10::optional<torch::Tensor> status, int64_t num_sms, c10::optional<torch::Tensor> stats,
               c10::optional<torch::Tensor> x_rows, c10::optional<torch::Tensor> ok, std::vector<torch::Tensor> wire_t) {
    TORCH_CHECK(gemm_t.size() == (bwd ? 11u : 6u) && layout.size() == 7 && send_t.size() == (bwd ? 6u : 7u) && sym_t.size() == 5 &&
                (offs.size() == 8 || offs.size() == 9) && push_t.size() == 3 && red_t.size() == (bwd ? 4u : 2u) && work_t.size() == 4 &&
                (wire_t.empty() || (wire_t.size() == 2 && offs.size() == 9)),
                "moe_layer: wrong argument lists");
    const torch::Tensor& slot_x = gemm_t[0];
    const int S = (int)slot_x.size(0), H = (int)slot_x.size(1);
    tmoe::LayerParams p{};
    p.bwd = bwd ? 1 : 0;
    p.H = H;
    p.El = (int)gemm_t[1].size(0);
    p.I = bwd ? (int)gemm_t[1].size(2) : (int)gemm_t[1].size(1) / 2;
    p.slot_rows = S;
    const int R = (int)gemm_t[3].size(0);
    p.out_rows = R;
    const TopK tk = topk(send_t[1]);
    p.T = tk.T; p.K = tk.K; p.E = (int)E; p.N = (int)N; p.rank = (int)rank;
    p.slot_x = bf16(slot_x, "slot_x");
    p.w1 = bf16(gemm_t[1], "w1");
    p.w2 = bf16(gemm_t[2], "w2");
    p.out0 = bf16(gemm_t[3], "out0");
    p.out1 = bf16(gemm_t[4], "out1");
    p.row_w = f32(gemm_t[5], "row_w");
    TORCH_CHECK(R > 0 && R % 128 == 0 && R <= S && gemm_t[4].size(0) == R && gemm_t[5].numel() >= R, "moe_layer: outputs need a multiple of 128 rows");
    if (bwd) {
        p.preact = bf16(gemm_t[6], "preact");
        p.droute_part = f32(gemm_t[7], "droute_part");
        p.xperm = bf16(gemm_t[8], "xperm");
        p.dw_down = bf16(gemm_t[9], "dW_down");
        p.dw_gateup = bf16(gemm_t[10], "dW_gateup");
        TORCH_CHECK(gemm_t[6].size(0) >= R && gemm_t[7].size(0) >= R && gemm_t[8].size(0) == R, "moe_layer: backward operands need one row per output row");
    }
    check_i32(layout[0], "mblock_expert");
    p.lay.mblock_expert = layout[0].data_ptr<int>();
    p.lay.num_mblocks_dev = i32(layout[1], "num_mblocks");
    p.lay.max_mblocks = R / 128;
    p.lay.unit_blk = i32(layout[2], "unit_blk");
    p.lay.num_units_dev = i32(layout[3], "num_units");
    p.lay.max_units = (int)layout[2].numel() - 1;
    p.seg_offsets = i32(layout[4], "seg_offsets");
    p.expert_total_local = i32(layout[5], "expert_total_local");
    p.unit_order = i32(layout[6], "unit_order");
    TORCH_CHECK(layout[0].numel() >= R / 128 && layout[6].numel() >= p.lay.max_units && layout[4].numel() == p.El + 1, "moe_layer: layout sizes");
    p.work = i32(work_t[0], "work");
    p.max_work = (int)(work_t[0].numel() / 4);
    p.num_work = i32(work_t[1], "num_work");
    p.expert_units = i32(work_t[2], "expert_units");
    p.sync = i32(work_t[3], "sync");
    TORCH_CHECK(work_t[2].numel() >= 2 * p.El && work_t[3].numel() >= 8 + p.lay.max_units, "moe_layer: work tensors too small");
    TORCH_CHECK(p.max_work >= tmoe::moe_layer_max_work(p.bwd, p.lay.max_units, H, p.I, p.El, p.T, (int)reduce_chunk), "moe_layer: work list too small");
    p.group_units = (int)group_units;
    p.lag_percent = (int)lag_percent;
    p.min_lag_items = (int)min_lag_items;
    p.reduce_chunk = (int)reduce_chunk;
    p.push.arena_ptrs = u64(sym_t[0], "arena_ptrs");
    p.push.landing_off = (uint64_t)offs[6];
    p.push.slot_tk = i32(push_t[0], "slot_tk");
    p.push.slot_row = i32(push_t[1], "slot_row");
    p.push.recv_row_base = i32(push_t[2], "recv_row_base");
    p.push.num_ranks = (int)N;
    TORCH_CHECK(push_t[0].numel() >= R && push_t[1].numel() >= R && push_t[2].numel() == N + 1 && sym_t[0].numel() == N, "moe_layer: push tables");
    p.gtw_off = bwd ? (uint64_t)offs[7] : 0;
    p.signal_ptrs = u64(sym_t[3], "signal_ptrs");
    p.my_signal = i32(sym_t[4], "my_signal");
    p.epoch = (int)epoch;
    p.landing = bf16(red_t[0], "landing");
    p.out = bf16(red_t[1], "out");
    TORCH_CHECK(red_t[0].size(0) >= (int64_t)tk.T * tk.K && red_t[0].size(1) == H && red_t[1].size(0) == tk.T && red_t[1].size(1) == H, "moe_layer: reduce shapes");
    if (bwd) {
        p.gtw_in = f32(red_t[2], "gtw_in");
        p.gtw_out = f32(red_t[3], "gtw_out");
        TORCH_CHECK(red_t[2].numel() >= (int64_t)tk.T * tk.K && red_t[3].numel() == (int64_t)tk.T * tk.K, "moe_layer: route gradient shapes");
    }
    tmoe::FusedArgs& f = p.f;
    f.num_dispatch_clusters = (int)num_dispatch_clusters;
    f.x = bf16(send_t[0], "x");
    f.topk_idx = tk.ptr;
    f.idx_is64 = tk.is64;
    f.send_order = i32(send_t[2], "send_order");
    f.num_send = i32(send_t[3], "num_send");
    f.max_send = (int)send_t[2].numel();
    f.send_slot = i32(send_t[4], "send_slot");
    f.send_row = i32(send_t[5], "send_row");
    f.topk_w = bwd ? nullptr : f32(send_t[6], "topk_w");
    f.T = tk.T; f.K = tk.K; f.H = H; f.E = (int)E; f.N = (int)N;
    f.with_meta = bwd ? 0 : 1;
    f.slot_cap = S;
    f.arena_ptrs = u64(sym_t[0], "arena_ptrs");
    f.ctrl_ptrs = u64(sym_t[1], "ctrl_ptrs");
    f.blk_cnt = i32(sym_t[2], "blk_cnt");
    f.unit_order = p.unit_order;
    f.seg_offsets = p.seg_offsets;
    f.expert_total_local = p.expert_total_local;
    f.off_slot_x = offs[0]; f.off_slot_w = offs[1]; f.off_slot_tk = offs[2]; f.off_slot_row = offs[3]; f.off_row_first = offs[4];
    f.off_blk_cnt = offs[5];
    TORCH_CHECK(send_t[0].size(1) == H && send_t[0].size(0) == tk.T && S % 128 == 0 && sym_t[2].numel() >= S / 128, "moe_layer: shape mismatch");
    TORCH_CHECK(bwd ? (gemm_t[6].size(1) == 2 * p.I) : true, "moe_layer: preact shape");
    if (!wire_t.empty()) {
        f.wire_rank = 1;
        f.slot_src = i32(wire_t[0], "slot_src");
        f.blk_ready = i32(wire_t[1], "blk_ready");
        f.off_slot_src = (uint64_t)offs[8];
        TORCH_CHECK(wire_t[0].numel() >= S && wire_t[1].numel() >= S / 128 && offs[8] >= 0 && offs[8] % 16 == 0, "moe_layer: wire tables");
    }
    p.status = opt_status(status);
    p.num_sms = (int)num_sms;
    if (ok.has_value()) p.geom_ok = i32(*ok, "ok");
    if (bwd && x_rows.has_value()) {
        // the kernel rebuilds X in slot space (gemm_t[8]) from one row per received token while the first GEMMs run
        TORCH_CHECK(x_rows->dim() == 2 && x_rows->size(1) == H, "x_rows must be [rows, H]");
        p.x_rows = bf16(*x_rows, "x_rows");
        p.expand_rows = R;
    }
    if (stats.has_value()) {
        TORCH_CHECK(stats->is_cuda() && stats->scalar_type() == torch::kInt64 && stats->is_contiguous() && stats->numel() >= tmoe::kLayerStatWords,
                    "stats must be a contiguous int64 CUDA tensor of 24 words");
        p.stats = reinterpret_cast<unsigned long long*>(stats->data_ptr<int64_t>());
    }
    c10::cuda::CUDAGuard guard(slot_x.device());
    TM_CHECK_CUDA(tmoe::moe_layer_launch(p, cur_stream()));
}

// The scheduler kernel of the whole-layer kernel alone (tests read the list back).
void moe_layer_schedule(bool bwd, int64_t H, int64_t I, int64_t T, torch::Tensor unit_order, torch::Tensor num_units, torch::Tensor seg_offsets,
                        torch::Tensor unit_blk, torch::Tensor mblock_expert, torch::Tensor expert_total_local, int64_t group_units, int64_t lag_percent, int64_t min_lag_items, int64_t reduce_chunk, torch::Tensor work,
                        torch::Tensor num_work, torch::Tensor expert_units) {
    tmoe::LayerParams p{};
    p.bwd = bwd ? 1 : 0;
    p.H = (int)H; p.I = (int)I; p.T = (int)T;
    p.El = (int)seg_offsets.numel() - 1;
    p.unit_order = i32(unit_order, "unit_order");
    p.lay.num_units_dev = i32(num_units, "num_units");
    p.lay.max_units = (int)unit_order.numel();
    p.seg_offsets = i32(seg_offsets, "seg_offsets");
    p.lay.unit_blk = i32(unit_blk, "unit_blk");
    p.lay.mblock_expert = i32(mblock_expert, "mblock_expert");
    p.expert_total_local = i32(expert_total_local, "expert_total_local");
    TORCH_CHECK(unit_blk.numel() >= unit_order.numel() + 1 && expert_total_local.numel() == p.El, "moe_layer_schedule: table sizes");
    p.group_units = (int)group_units; p.lag_percent = (int)lag_percent; p.min_lag_items = (int)min_lag_items; p.reduce_chunk = (int)reduce_chunk;
    p.work = i32(work, "work");
    p.max_work = (int)(work.numel() / 4);
    p.num_work = i32(num_work, "num_work");
    p.expert_units = i32(expert_units, "expert_units");
    TORCH_CHECK(expert_units.numel() >= 2 * p.El, "expert_units too small");
    c10::cuda::CUDAGuard guard(work.device());
    TM_CHECK_CUDA(tmoe::moe_layer_schedule(p, cur_stream()));
}

int64_t moe_layer_max_work(bool bwd, int64_t max_units, int64_t H, int64_t I, int64_t El, int64_t T, int64_t reduce_chunk) {
    return tmoe::moe_layer_max_work(bwd ? 1 : 0, (int)max_units, (int)H, (int)I, (int)El, (int)T, (int)reduce_chunk);
}

void ep_barrier(torch::Tensor signal_ptrs, int64_t rank, int64_t N, int64_t epoch, c10::optional<torch::Tensor> status, int64_t site,
                int64_t limit_ms, int64_t mode, c10::optional<torch::Tensor> mask) {
    c10::cuda::CUDAGuard guard(signal_ptrs.device());
    TM_CHECK_CUDA(tmoe::ep_barrier(u64(signal_ptrs, "signal_ptrs"), (int)rank, (int)N, (int)epoch, opt_status(status), (int)site,
                                   (int)limit_ms, (int)mode, mask.has_value() ? i32(*mask, "mask") : nullptr, cur_stream()));
}

void dispatch_push(torch::Tensor x, torch::Tensor topk_idx, torch::Tensor topk_w, int64_t E, int64_t N, torch::Tensor send_slot,
                   torch::Tensor send_row, torch::Tensor land_off, torch::Tensor arena_ptrs, std::vector<int64_t> offsets,
                   bool with_meta, int64_t num_blocks, c10::optional<torch::Tensor> ok) {
    const TopK tk = topk(topk_idx);
    TORCH_CHECK(x.dim() == 2 && x.size(0) == tk.T, "x must be [T,H]");
    c10::cuda::CUDAGuard guard(x.device());
    TM_CHECK_CUDA(tmoe::dispatch_push(bf16(x, "x"), tk.ptr, tk.is64, f32(topk_w, "topk_weights"), tk.T, tk.K, (int)x.size(1), (int)E, (int)N,
                                      i32(send_slot, "send_slot"), i32(send_row, "send_row"), i32(land_off, "land_off"),
                                      u64(arena_ptrs, "arena_ptrs"), sym_offsets(offsets), with_meta ? 1 : 0, (int)num_blocks,
                                      ok.has_value() ? i32(*ok, "ok") : nullptr, cur_stream()));
}

void tail_fill(torch::Tensor x, torch::Tensor idx, torch::Tensor w, torch::Tensor rows_dev) {
    TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == torch::kInt64 && idx.is_contiguous() && idx.dim() == 2 && idx.size(0) == x.size(0) &&
                w.sizes() == idx.sizes(), "tail_fill: idx must be int64 [rows, K] and w fp32 [rows, K]");
    c10::cuda::CUDAGuard guard(x.device());
    TM_CHECK_CUDA(tmoe::tail_fill(bf16(x, "x"), idx.data_ptr<int64_t>(), f32(w, "w"), i32(rows_dev, "rows"), (int)x.size(0), (int)x.size(1),
                                  (int)idx.size(1), cur_stream()));
}

void expand_rows(torch::Tensor rows, torch::Tensor slot_row, torch::Tensor out, int64_t num_slots) {
    TORCH_CHECK(out.dim() == 2 && out.size(0) >= num_slots && slot_row.numel() >= num_slots && rows.size(1) == out.size(1),
                "expand_rows: shape mismatch");
    c10::cuda::CUDAGuard guard(out.device());
    TM_CHECK_CUDA(tmoe::expand_rows(bf16(rows, "rows"), i32(slot_row, "slot_row"), bf16(out, "out"), (int)num_slots, (int)out.size(1),
                                    cur_stream()));
}

void combine_push(torch::Tensor y, torch::Tensor row_slots, torch::Tensor row_land, torch::Tensor recv_row_base, int64_t R, int64_t N,
                  torch::Tensor arena_ptrs, std::vector<int64_t> offsets, c10::optional<torch::Tensor> droute_part,
                  c10::optional<torch::Tensor> slot_tk, bool with_payload, int64_t num_blocks) {
    TORCH_CHECK(row_slots.dim() == 2 && row_slots.size(0) >= R, "row_slots must be [rows,K]");
    const float* dp = nullptr;
    const int* stk = nullptr;
    int n_parts = 0;
    if (droute_part.has_value()) {
        TORCH_CHECK(slot_tk.has_value(), "slot_tk is required with droute_part");
        dp = f32(*droute_part, "droute_part");
        n_parts = (int)droute_part->size(1);
        stk = i32(*slot_tk, "slot_tk");
    }
    c10::cuda::CUDAGuard guard(y.device());
    TM_CHECK_CUDA(tmoe::combine_push(bf16(y, "y"), i32(row_slots, "row_slots"), i32(row_land, "row_land"),
                                     i32(recv_row_base, "recv_row_base"), (int)R, (int)row_slots.size(1), (int)y.size(1), (int)N,
                                     u64(arena_ptrs, "arena_ptrs"), sym_offsets(offsets), dp, n_parts, stk, with_payload ? 1 : 0, (int)num_blocks,
                                     cur_stream()));
}

void combine_reduce(torch::Tensor landing, torch::Tensor land_off, torch::Tensor ndst, torch::Tensor out) {
    c10::cuda::CUDAGuard guard(out.device());
    TM_CHECK_CUDA(tmoe::combine_reduce(bf16(landing, "landing"), i32(land_off, "land_off"), i32(ndst, "ndst"), bf16(out, "out"),
                                       (int)out.size(0), (int)out.size(1), cur_stream()));
}

void slot_rows_push(torch::Tensor y, torch::Tensor slot_tk, torch::Tensor slot_row, torch::Tensor recv_row_base, int64_t S,
                    torch::Tensor arena_ptrs, int64_t landing_off) {
    TORCH_CHECK(y.dim() == 2 && y.size(0) >= S && slot_tk.numel() >= S && slot_row.numel() >= S, "slot_rows_push: shapes");
    c10::cuda::CUDAGuard guard(y.device());
    TM_CHECK_CUDA(tmoe::slot_rows_push(bf16(y, "y"), i32(slot_tk, "slot_tk"), i32(slot_row, "slot_row"), i32(recv_row_base, "recv_row_base"),
                                       (int)S, (int)y.size(1), (int)arena_ptrs.numel(), u64(arena_ptrs, "arena_ptrs"), (uint64_t)landing_off,
                                       cur_stream()));
}

void combine_reduce_slots(torch::Tensor landing, torch::Tensor topk_idx, int64_t E, torch::Tensor out, c10::optional<torch::Tensor> weights) {
    const TopK tk = topk(topk_idx);
    TORCH_CHECK(out.dim() == 2 && out.size(0) == tk.T && landing.size(0) >= (int64_t)tk.T * tk.K && landing.size(1) == out.size(1),
                "combine_reduce_slots: shape mismatch");
    c10::cuda::CUDAGuard guard(out.device());
    TM_CHECK_CUDA(tmoe::combine_reduce_slots(bf16(landing, "landing"), tk.ptr, tk.is64, bf16(out, "out"), tk.T, tk.K, (int)out.size(1), (int)E,
                                             weights.has_value() ? f32(*weights, "weights") : nullptr, cur_stream()));
}

void droute_push(torch::Tensor droute_part, torch::Tensor slot_tk, torch::Tensor slot_row, torch::Tensor recv_row_base, int64_t S,
                 torch::Tensor arena_ptrs, int64_t gtw_off) {
    TORCH_CHECK(droute_part.dim() == 2 && droute_part.size(0) >= S && slot_tk.numel() >= S && slot_row.numel() >= S, "droute_push: shapes");
    c10::cuda::CUDAGuard guard(droute_part.device());
    TM_CHECK_CUDA(tmoe::droute_push(f32(droute_part, "droute_part"), (int)droute_part.size(1), i32(slot_tk, "slot_tk"),
                                    i32(slot_row, "slot_row"), i32(recv_row_base, "recv_row_base"), (int)S, (int)arena_ptrs.numel(),
                                    u64(arena_ptrs, "arena_ptrs"), (uint64_t)gtw_off, cur_stream()));
}

torch::Tensor numerics_check(torch::Tensor a, torch::Tensor b) {
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.is_contiguous() && b.is_contiguous() && a.numel() == b.numel() &&
                a.scalar_type() == b.scalar_type(), "numerics_check: two contiguous CUDA tensors of one dtype and size");
    TORCH_CHECK(a.scalar_type() == torch::kBFloat16 || a.scalar_type() == torch::kFloat32, "numerics_check: bf16 or fp32");
    c10::cuda::CUDAGuard guard(a.device());
    auto out = torch::empty({6}, torch::TensorOptions().dtype(torch::kFloat64).device(a.device()));
    TM_CHECK_CUDA(tmoe::numerics_check(a.data_ptr(), b.data_ptr(), a.numel(), a.scalar_type() == torch::kBFloat16 ? 1 : 0,
                                       out.data_ptr<double>(), cur_stream()));
    return out;
}

// ---- low-latency kernels (lowlat.cu).  `geom` = [num_ranks, rank, num_experts, max_tokens, hidden, use_fp8, use_ue8m0, round_scale,
// use_logfmt, off_d_stage, off_d_flags, off_c_stage, off_c_flags, d_msg_bytes, c_row_bytes]
tmoe::LowLatLayout ll_layout(const std::vector<int64_t>& g) {
    TORCH_CHECK(g.size() == 15, "low-latency geometry needs 15 numbers");
    tmoe::LowLatLayout l{};
    l.num_ranks = (int)g[0]; l.rank = (int)g[1]; l.num_experts = (int)g[2]; l.max_tokens = (int)g[3]; l.hidden = (int)g[4];
    l.use_fp8 = (int)g[5]; l.use_ue8m0 = (int)g[6]; l.round_scale = (int)g[7]; l.use_logfmt = (int)g[8];
    l.off_d_stage = (uint64_t)g[9]; l.off_d_flags = (uint64_t)g[10]; l.off_c_stage = (uint64_t)g[11]; l.off_c_flags = (uint64_t)g[12];
    l.d_msg_bytes = (uint32_t)g[13]; l.c_row_bytes = (uint32_t)g[14];
    return l;
}
int* opt_i32(const c10::optional<torch::Tensor>& t, const char* name) { return t.has_value() ? i32(*t, name) : nullptr; }
long long* opt_i64(const c10::optional<torch::Tensor>& t, const char* name) {
    if (!t.has_value()) return nullptr;
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kInt64 && t->is_contiguous(), name, " must be a contiguous int64 CUDA tensor");
    return reinterpret_cast<long long*>(t->data_ptr<int64_t>());
}

void ll_dispatch_send(std::vector<int64_t> geom, torch::Tensor x, torch::Tensor topk_idx, torch::Tensor arena_ptrs, int64_t call_seq,
                      c10::optional<torch::Tensor> mask) {
    const TopK tk = topk(topk_idx);
    const auto lay = ll_layout(geom);
    TORCH_CHECK(x.dim() == 2 && x.size(0) == tk.T && x.size(1) == lay.hidden, "x must be [T, hidden]");
    c10::cuda::CUDAGuard guard(x.device());
    TM_CHECK_CUDA(tmoe::ll_dispatch_send(lay, bf16(x, "x"), tk.ptr, tk.is64, tk.T, tk.K, u64(arena_ptrs, "arena_ptrs"), call_seq,
                                         opt_i32(mask, "mask"), cur_stream()));
}

void ll_dispatch_recv(std::vector<int64_t> geom, torch::Tensor arena_local, torch::Tensor recv_x, c10::optional<torch::Tensor> recv_scales,
                      torch::Tensor src_info, torch::Tensor layout_range, torch::Tensor recv_count, c10::optional<torch::Tensor> expert_stats,
                      c10::optional<torch::Tensor> wait_stats, int64_t call_seq, c10::optional<torch::Tensor> mask, bool shrink,
                      int64_t limit_ms, c10::optional<torch::Tensor> status) {
    const auto lay = ll_layout(geom);
    const int El = lay.num_experts / lay.num_ranks;
    const int64_t NM = (int64_t)lay.num_ranks * lay.max_tokens;
    TORCH_CHECK(recv_x.is_cuda() && recv_x.is_contiguous() && recv_x.numel() == El * NM * lay.hidden, "recv_x must be [E_local, ranks*max_tokens, hidden]");
    TORCH_CHECK(!lay.use_fp8 || (recv_scales.has_value() && recv_scales->is_cuda()), "FP8 dispatch needs a scales tensor");
    TORCH_CHECK(src_info.numel() == El * NM && layout_range.numel() == El * lay.num_ranks && recv_count.numel() == El, "low-latency receive tensors");
    c10::cuda::CUDAGuard guard(recv_x.device());
    TM_CHECK_CUDA(tmoe::ll_dispatch_recv(lay, arena_local.data_ptr(), recv_x.data_ptr(), recv_scales.has_value() ? recv_scales->data_ptr() : nullptr,
                                         i32(src_info, "src_info"), opt_i64(layout_range, "layout_range"), i32(recv_count, "recv_count"),
                                         opt_i32(expert_stats, "expert_stats"), opt_i64(wait_stats, "wait_stats"), call_seq, opt_i32(mask, "mask"),
                                         shrink ? 1 : 0, (uint64_t)limit_ms * 1000000ull, opt_status(status), cur_stream()));
}

void ll_combine_send(std::vector<int64_t> geom, torch::Tensor x, torch::Tensor src_info, torch::Tensor layout_range, torch::Tensor arena_ptrs,
                     int64_t call_seq, c10::optional<torch::Tensor> mask) {
    const auto lay = ll_layout(geom);
    const int El = lay.num_experts / lay.num_ranks;
    TORCH_CHECK(x.numel() == (int64_t)El * lay.num_ranks * lay.max_tokens * lay.hidden, "x must be [E_local, ranks*max_tokens, hidden]");
    c10::cuda::CUDAGuard guard(x.device());
    TM_CHECK_CUDA(tmoe::ll_combine_send(lay, bf16(x, "x"), i32(src_info, "src_info"), opt_i64(layout_range, "layout_range"),
                                        u64(arena_ptrs, "arena_ptrs"), call_seq, opt_i32(mask, "mask"), cur_stream()));
}

void ll_combine_recv(std::vector<int64_t> geom, torch::Tensor arena_local, torch::Tensor topk_idx, torch::Tensor topk_weights, torch::Tensor out,
                     c10::optional<torch::Tensor> wait_stats, int64_t call_seq, c10::optional<torch::Tensor> mask, bool shrink, int64_t limit_ms,
                     c10::optional<torch::Tensor> status) {
    const TopK tk = topk(topk_idx);
    const auto lay = ll_layout(geom);
    TORCH_CHECK(out.dim() == 2 && out.size(0) == tk.T && out.size(1) == lay.hidden && topk_weights.numel() == (int64_t)tk.T * tk.K, "combine shapes");
    c10::cuda::CUDAGuard guard(out.device());
    TM_CHECK_CUDA(tmoe::ll_combine_recv(lay, arena_local.data_ptr(), tk.ptr, tk.is64, f32(topk_weights, "topk_weights"), tk.T, tk.K, bf16(out, "out"),
                                        opt_i64(wait_stats, "wait_stats"), call_seq, opt_i32(mask, "mask"), shrink ? 1 : 0,
                                        (uint64_t)limit_ms * 1000000ull, opt_status(status), cur_stream()));
}

void ll_mask_update(torch::Tensor mask, int64_t rank, int64_t value) {
    c10::cuda::CUDAGuard guard(mask.device());
    TM_CHECK_CUDA(tmoe::ll_mask_update(i32(mask, "mask"), (int)mask.numel(), (int)rank, (int)value, cur_stream()));
}
void ll_mask_query(torch::Tensor mask, torch::Tensor out) {
    TORCH_CHECK(out.numel() >= mask.numel(), "mask_status too small");
    c10::cuda::CUDAGuard guard(mask.device());
    TM_CHECK_CUDA(tmoe::ll_mask_query(i32(mask, "mask"), (int)mask.numel(), i32(out, "mask_status"), cur_stream()));
}
void ll_mask_clean(torch::Tensor mask) {
    c10::cuda::CUDAGuard guard(mask.device());
    TM_CHECK_CUDA(tmoe::ll_mask_clean(i32(mask, "mask"), (int)mask.numel(), cur_stream()));
}

// Tensor view over a range of the local arena.
torch::Tensor arena_view(tmoe::SymmetricArena& arena, int64_t offset, std::vector<int64_t> sizes, py::object dtype) {
    const auto st = torch::python::detail::py_object_to_dtype(dtype);
    int64_t n = 1;
    for (auto s : sizes) n *= s;
    TORCH_CHECK(offset >= 0 && offset % 16 == 0, "arena view offset must be a non-negative multiple of 16");
    TORCH_CHECK((size_t)(offset + n * (int64_t)c10::elementSize(st)) <= arena.bytes(), "arena view out of range");
    int dev = 0;
    cudaGetDevice(&dev);
    return torch::from_blob(reinterpret_cast<void*>(arena.local_ptr() + offset), sizes,
                            torch::TensorOptions().dtype(st).device(torch::kCUDA, dev));
}

}  // namespace

void register_more(pybind11::module_& m) {
    m.def("route_chunk_tokens", &tmoe::route_chunk_tokens);
    m.def("route_hist", &route_hist, py::arg("topk_idx"), py::arg("E"), py::arg("N"), py::arg("chunk_hist"), py::arg("in_rank") = py::none());
    m.def("route_sum", &route_sum);
    m.def("route_scan", &route_scan);
    m.def("layout_finalize", &layout_finalize, py::arg("meta"), py::arg("rank"), py::arg("N"), py::arg("E"), py::arg("layout"),
          py::arg("cap_rows") = 0, py::arg("cap_slots") = 0, py::arg("cap_tokens") = 0);
    m.def("slot_pad_fill", &slot_pad_fill, py::arg("seg_offsets"), py::arg("expert_total_local"), py::arg("slot_row"), py::arg("slot_w"),
          py::arg("slot_tk"), py::arg("mblock_expert"), py::arg("unit_blk"), py::arg("num_units"), py::arg("ok") = py::none());
    m.def("route_assign", &route_assign);
    m.def("arrival_order", &arrival_order, py::arg("meta"), py::arg("rank"), py::arg("N"), py::arg("E"), py::arg("groups"), py::arg("seg_offsets"),
          py::arg("unit_blk"), py::arg("num_units"), py::arg("blk_group"), py::arg("unit_order"), py::arg("ok") = py::none());
    m.def("zero_pad_rows", &zero_pad_rows, py::arg("seg_offsets"), py::arg("expert_total_local"), py::arg("slot_x"), py::arg("ok") = py::none());
    m.def("fused_dispatch_gemm", &fused_dispatch_gemm);
    m.def("moe_layer", &moe_layer, py::arg("bwd"), py::arg("gemm_t"), py::arg("layout"), py::arg("send_t"), py::arg("sym_t"), py::arg("offs"),
          py::arg("push_t"), py::arg("red_t"), py::arg("work_t"), py::arg("E"), py::arg("N"), py::arg("rank"), py::arg("epoch"),
          py::arg("num_dispatch_clusters"), py::arg("group_units"), py::arg("lag_percent"), py::arg("min_lag_items"), py::arg("reduce_chunk"),
          py::arg("status"), py::arg("num_sms"), py::arg("stats"), py::arg("x_rows"), py::arg("ok"),
          py::arg("wire_t") = std::vector<torch::Tensor>());
    m.def("moe_layer_max_work", &moe_layer_max_work);
    m.def("moe_layer_schedule", &moe_layer_schedule);
    m.def("ep_barrier", &ep_barrier, py::arg("signal_ptrs"), py::arg("rank"), py::arg("N"), py::arg("epoch"), py::arg("status"),
          py::arg("site"), py::arg("limit_ms"), py::arg("mode") = 0, py::arg("mask") = py::none());
    m.def("dispatch_push", &dispatch_push, py::arg("x"), py::arg("topk_idx"), py::arg("topk_w"), py::arg("E"), py::arg("N"), py::arg("send_slot"),
          py::arg("send_row"), py::arg("land_off"), py::arg("arena_ptrs"), py::arg("offsets"), py::arg("with_meta"), py::arg("num_blocks"),
          py::arg("ok") = py::none());
    m.def("tail_fill", &tail_fill);
    m.def("expand_rows", &expand_rows);
    m.def("combine_push", &combine_push);
    m.def("combine_reduce", &combine_reduce);
    m.def("combine_reduce_slots", &combine_reduce_slots);
    m.def("slot_rows_push", &slot_rows_push);
    m.def("droute_push", &droute_push);
    m.def("numerics_check", &numerics_check);
    m.def("ll_dispatch_send", &ll_dispatch_send);
    m.def("ll_dispatch_recv", &ll_dispatch_recv);
    m.def("ll_combine_send", &ll_combine_send);
    m.def("ll_combine_recv", &ll_combine_recv);
    m.def("ll_mask_update", &ll_mask_update);
    m.def("ll_mask_query", &ll_mask_query);
    m.def("ll_mask_clean", &ll_mask_clean);

    py::class_<tmoe::SymmetricArena>(m, "SymmetricArena")
        .def(py::init<int, int, size_t, bool, bool>(), py::arg("rank"), py::arg("world"), py::arg("bytes"), py::arg("vmm") = false,
             py::arg("fabric") = false)
        .def("export_fd", &tmoe::SymmetricArena::export_fd)
        .def("open_peer_fds", &tmoe::SymmetricArena::open_peer_fds)
        .def("is_vmm", &tmoe::SymmetricArena::is_vmm)
        .def("has_fabric_handle", &tmoe::SymmetricArena::has_fabric_handle)
        .def("export_handle", [](const tmoe::SymmetricArena& a) { return py::bytes(a.export_handle()); })
        .def("open_peers",
             [](tmoe::SymmetricArena& a, const std::vector<py::bytes>& hs) {
                 std::vector<std::string> v;
                 for (const auto& h : hs) v.emplace_back(static_cast<std::string>(h));
                 a.open_peers(v);
             })
        .def("adopt_peer_pointers", &tmoe::SymmetricArena::adopt_peer_pointers)
        .def("close", &tmoe::SymmetricArena::close)
        .def("local_ptr", &tmoe::SymmetricArena::local_ptr)
        .def("peer_ptrs", &tmoe::SymmetricArena::peer_ptrs)
        .def("bytes", &tmoe::SymmetricArena::bytes)
        .def("is_open", &tmoe::SymmetricArena::is_open)
        .def("view", &arena_view);
}
