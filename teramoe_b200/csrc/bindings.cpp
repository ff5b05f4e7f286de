// Python bindings (module teramoe_b200_C).  Thin: argument checks + raw-pointer calls into the
// launchers declared in gemm.h / routing.h / comm.h / runtime.h.  No kernel code here.
//
// Reference counterpart: the pybind block at csrc/moe_extension.cpp:2573-2657.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "gemm.h"
#include "launch_count.h"

namespace {

#define TM_CHECK_CUDA(call)                                                                          \
    do {                                                                                             \
        tmoe::count_launch();                                                                        \
        cudaError_t _e = (call);                                                                     \
        TORCH_CHECK(_e == cudaSuccess, "teramoe_b200: ", #call, " failed: ", cudaGetErrorString(_e)); \
    } while (0)

void check_bf16(const torch::Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(t.scalar_type() == torch::kBFloat16, name, " must be bf16");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}
void check_i32(const torch::Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kInt32 && t.is_contiguous(), name, " must be a contiguous int32 CUDA tensor");
}
void check_f32(const torch::Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kFloat32 && t.is_contiguous(), name, " must be a contiguous fp32 CUDA tensor");
}
int* status_ptr(const c10::optional<torch::Tensor>& status) {
    if (!status.has_value()) return nullptr;
    check_i32(*status, "status");
    TORCH_CHECK(status->numel() >= 8, "status must hold 8 ints");
    return status->data_ptr<int>();
}
cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

// Python passes the block layout as [mblock_expert, num_mblocks] or, for the CTA-pair kernels,
// [mblock_expert, num_mblocks, unit_blk, num_units].
tmoe::MGroupLayout make_layout(const std::vector<torch::Tensor>& t, int S) {
    TORCH_CHECK(t.size() == 2 || t.size() == 4, "layout must be [mblock_expert, num_mblocks] (+ [unit_blk, num_units])");
    tmoe::MGroupLayout lay;
    check_i32(t[0], "mblock_expert"); check_i32(t[1], "num_mblocks");
    TORCH_CHECK(S % 128 == 0 && t[0].numel() >= S / 128, "mblock_expert too small");
    lay.mblock_expert = t[0].data_ptr<int>();
    lay.num_mblocks_dev = t[1].data_ptr<int>();
    lay.max_mblocks = S / 128;
    if (t.size() == 4) {
        check_i32(t[2], "unit_blk"); check_i32(t[3], "num_units");
        TORCH_CHECK(t[2].numel() >= 2, "unit_blk too small");
        lay.unit_blk = t[2].data_ptr<int>();
        lay.num_units_dev = t[3].data_ptr<int>();
        lay.max_units = (int)t[2].numel() - 1;
    }
    return lay;
}

// Python passes the push target as ([arena_ptrs int64, slot_tk, slot_row, recv_row_base], landing_off).
bool make_push(const c10::optional<std::vector<torch::Tensor>>& t, int64_t landing_off, tmoe::PushTarget& p) {
    if (!t.has_value()) return false;
    TORCH_CHECK(t->size() == 4, "push target must be [arena_ptrs, slot_tk, slot_row, recv_row_base]");
    const auto& v = *t;
    TORCH_CHECK(v[0].is_cuda() && v[0].scalar_type() == torch::kInt64 && v[0].is_contiguous(), "arena_ptrs must be int64 CUDA");
    check_i32(v[1], "slot_tk"); check_i32(v[2], "slot_row"); check_i32(v[3], "recv_row_base");
    p.arena_ptrs = reinterpret_cast<const uint64_t*>(v[0].data_ptr<int64_t>());
    p.landing_off = (uint64_t)landing_off;
    p.slot_tk = v[1].data_ptr<int>();
    p.slot_row = v[2].data_ptr<int>();
    p.recv_row_base = v[3].data_ptr<int>();
    p.num_ranks = (int)v[0].numel();
    TORCH_CHECK(v[3].numel() == p.num_ranks + 1, "recv_row_base must have ranks + 1 entries");
    return true;
}

// ---- grouped GEMMs ------------------------------------------------------------------------------
void gemm_fwd_gateup(torch::Tensor xperm, torch::Tensor w_gateup, torch::Tensor act, torch::Tensor preact, torch::Tensor row_w,
                     std::vector<torch::Tensor> layout, c10::optional<torch::Tensor> gather_rows,
                     c10::optional<torch::Tensor> status, int64_t num_sms) {
    check_bf16(xperm, "xperm"); check_bf16(w_gateup, "w_gateup"); check_bf16(act, "act"); check_bf16(preact, "preact");
    check_f32(row_w, "row_w"); 
    const int H = xperm.size(1), E = w_gateup.size(0), I = w_gateup.size(1) / 2;
    const int S = gather_rows.has_value() ? (int)gather_rows->numel() : (int)xperm.size(0);
    const int* gr = nullptr;
    if (gather_rows.has_value()) { check_i32(*gather_rows, "gather_rows"); gr = gather_rows->data_ptr<int>(); }
    TORCH_CHECK(S % 128 == 0 && w_gateup.size(2) == H && act.size(0) == S && act.size(1) == I && preact.size(0) == S &&
                preact.size(1) == 2 * I && row_w.numel() == S, "gemm_fwd_gateup: shape mismatch");
    c10::cuda::CUDAGuard guard(xperm.device());
    TM_CHECK_CUDA(tmoe::gemm_fwd_gateup(xperm.data_ptr(), w_gateup.data_ptr(), act.data_ptr(), preact.data_ptr(), row_w.data_ptr<float>(),
                                        make_layout(layout, S), H, I, E, gr,
                                        (int)xperm.size(0), status_ptr(status), (int)num_sms, cur_stream()));
}

void gemm_fwd_down(torch::Tensor act, torch::Tensor w_down, c10::optional<torch::Tensor> y_opt, std::vector<torch::Tensor> layout,
                   c10::optional<torch::Tensor> status, int64_t num_sms, c10::optional<std::vector<torch::Tensor>> push, int64_t landing_off) {
    tmoe::PushTarget pt;
    const bool has_push = make_push(push, landing_off, pt);
    TORCH_CHECK(has_push || y_opt.has_value(), "gemm_fwd_down: need y or a push target");
    torch::Tensor y = y_opt.has_value() ? *y_opt : act;
    check_bf16(act, "act"); check_bf16(w_down, "w_down"); check_bf16(y, "y");
    const int S = act.size(0), I = act.size(1), E = w_down.size(0), H = w_down.size(1);
    TORCH_CHECK(S % 128 == 0 && w_down.size(2) == I && (has_push || (y.size(0) == S && y.size(1) == H)), "gemm_fwd_down: shape mismatch");
    if (has_push) TORCH_CHECK(push->at(1).numel() >= S && push->at(2).numel() >= S, "push tables too small");
    c10::cuda::CUDAGuard guard(act.device());
    TM_CHECK_CUDA(tmoe::gemm_fwd_down(act.data_ptr(), w_down.data_ptr(), y.data_ptr(), make_layout(layout, S), H, I, E, status_ptr(status), (int)num_sms, cur_stream(), has_push ? &pt : nullptr));
}

void gemm_bwd_gradact(torch::Tensor dyperm, torch::Tensor w_down, torch::Tensor preact, torch::Tensor row_w, torch::Tensor dgu,
                      torch::Tensor act_w, torch::Tensor droute_part, std::vector<torch::Tensor> layout,
                      c10::optional<torch::Tensor> gather_rows, c10::optional<torch::Tensor> status, int64_t num_sms) {
    check_bf16(dyperm, "dyperm"); check_bf16(w_down, "w_down"); check_bf16(preact, "preact"); check_bf16(dgu, "dgu"); check_bf16(act_w, "act_w");
    check_f32(row_w, "row_w"); check_f32(droute_part, "droute_part");
    
    const int H = dyperm.size(1), E = w_down.size(0), I = w_down.size(2);
    const int S = gather_rows.has_value() ? (int)gather_rows->numel() : (int)dyperm.size(0);
    const int* gr = nullptr;
    if (gather_rows.has_value()) { check_i32(*gather_rows, "gather_rows"); gr = gather_rows->data_ptr<int>(); }
    TORCH_CHECK(S % 128 == 0 && w_down.size(1) == H && preact.size(0) == S && preact.size(1) == 2 * I && dgu.size(0) == S &&
                dgu.size(1) == 2 * I && act_w.size(0) == S && act_w.size(1) == I && row_w.numel() == S &&
                droute_part.size(0) == S && droute_part.size(1) == tmoe::gemm_num_droute_parts(I),
                "gemm_bwd_gradact: shape mismatch");
    c10::cuda::CUDAGuard guard(dyperm.device());
    TM_CHECK_CUDA(tmoe::gemm_bwd_gradact(dyperm.data_ptr(), w_down.data_ptr(), preact.data_ptr(), row_w.data_ptr<float>(), dgu.data_ptr(),
                                         act_w.data_ptr(), droute_part.data_ptr<float>(), make_layout(layout, S), H, I, E, gr, (int)dyperm.size(0), status_ptr(status),
                                         (int)num_sms, cur_stream()));
}

void gemm_bwd_dx(torch::Tensor dgu, torch::Tensor w_gateup, c10::optional<torch::Tensor> dx_opt, std::vector<torch::Tensor> layout,
                 c10::optional<torch::Tensor> status, int64_t num_sms, c10::optional<std::vector<torch::Tensor>> push, int64_t landing_off) {
    tmoe::PushTarget pt;
    const bool has_push = make_push(push, landing_off, pt);
    TORCH_CHECK(has_push || dx_opt.has_value(), "gemm_bwd_dx: need dxperm or a push target");
    torch::Tensor dxperm = dx_opt.has_value() ? *dx_opt : dgu;
    check_bf16(dgu, "dgu"); check_bf16(w_gateup, "w_gateup"); check_bf16(dxperm, "dxperm");
    
    const int S = dgu.size(0), I = dgu.size(1) / 2, E = w_gateup.size(0), H = w_gateup.size(2);
    TORCH_CHECK(S % 128 == 0 && w_gateup.size(1) == 2 * I && (has_push || (dxperm.size(0) == S && dxperm.size(1) == H)),
                "gemm_bwd_dx: shape mismatch");
    if (has_push) TORCH_CHECK(push->at(1).numel() >= S && push->at(2).numel() >= S, "push tables too small");
    c10::cuda::CUDAGuard guard(dgu.device());
    TM_CHECK_CUDA(tmoe::gemm_bwd_dx(dgu.data_ptr(), w_gateup.data_ptr(), dxperm.data_ptr(), make_layout(layout, S), H, I, E, status_ptr(status), (int)num_sms, cur_stream(), has_push ? &pt : nullptr));
}

void gemm_wgrad(torch::Tensor a, torch::Tensor b, torch::Tensor dw, torch::Tensor seg_offsets, c10::optional<torch::Tensor> gather_rows,
                int64_t gather_operand, bool cta_pairs, c10::optional<torch::Tensor> status, int64_t num_sms) {
    check_bf16(a, "a"); check_bf16(b, "b"); check_bf16(dw, "dw"); check_i32(seg_offsets, "seg_offsets");
    const int M = a.size(1), N = b.size(1), E = dw.size(0);
    const int* gr = nullptr;
    int S, src_rows = 0;
    if (gather_rows.has_value() && gather_operand != 0) {
        check_i32(*gather_rows, "gather_rows");
        gr = gather_rows->data_ptr<int>();
        S = (int)gather_rows->numel();
        TORCH_CHECK(gather_operand == 1 || gather_operand == 2, "gather_operand must be 0, 1 or 2");
        src_rows = gather_operand == 1 ? (int)a.size(0) : (int)b.size(0);
        TORCH_CHECK((gather_operand == 1 ? b.size(0) : a.size(0)) == S, "gemm_wgrad: dense operand must have one row per slot");
    } else {
        gather_operand = 0;
        S = (int)a.size(0);
        TORCH_CHECK(b.size(0) == S, "gemm_wgrad: shape mismatch");
    }
    TORCH_CHECK(dw.size(1) == M && dw.size(2) == N && seg_offsets.numel() == E + 1, "gemm_wgrad: shape mismatch");
    c10::cuda::CUDAGuard guard(dw.device());
    TM_CHECK_CUDA(tmoe::gemm_wgrad(a.data_ptr(), b.data_ptr(), dw.data_ptr(), seg_offsets.data_ptr<int>(), S, M, N, E, gr,
                                   (int)gather_operand, src_rows, cta_pairs, status_ptr(status), (int)num_sms, cur_stream()));
}

}  // namespace

void register_more(pybind11::module_& m);  // routing / comm / runtime bindings (bindings_more.cpp)

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "teramoe_b200 native kernels (sm_100a)";
    m.def("gemm_fwd_gateup", &gemm_fwd_gateup);
    m.def("gemm_fwd_down", &gemm_fwd_down);
    m.def("gemm_bwd_gradact", &gemm_bwd_gradact);
    m.def("gemm_bwd_dx", &gemm_bwd_dx);
    m.def("gemm_wgrad", &gemm_wgrad);
    m.def("gemm_num_droute_parts", &tmoe::gemm_num_droute_parts);
    m.def("gemm_has_gather4", &tmoe::gemm_has_gather4);
    m.def("launch_count", [] { return tmoe::launch_counter().load(); });
    register_more(m);
}
