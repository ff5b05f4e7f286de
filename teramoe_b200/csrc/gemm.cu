// Persistent, warp-specialised tcgen05 grouped GEMM family for the expert MLP.
//
// One kernel template covers the five contractions of a SwiGLU expert layer:
//   forward   GU  = X . Wgu^T   (+ SwiGLU * route epilogue, pre-activation side store)
//   forward   Y   = Act . Wd^T
//   backward  gA  = dY . Wd     (B read MN-major straight from the forward layout; dSwiGLU epilogue)
//   backward  dX  = dGU . Wgu   (B MN-major)
//   backward  dW  = A^T . B     (both operands MN-major, K = the expert's rows, variable per expert)
//
// CTA layout (384 threads, one CTA per SM, 1-CTA UMMA 128x256x16):
//   warp 0      TMA producer (one elected lane)        4-stage ring, 48 KB per stage
//   warp 1      UMMA issuer  (one elected lane)        accumulators double-buffered in TMEM (2 x 256 cols)
//   warp 2      tensor-memory allocation / release
//   warp 3      idle
//   warps 4-11  epilogue: warp w reads TMEM lanes 32*(w%4).. and column half (w-4)/4
//
// All waits are bounded (ptx.cuh).  Tiles never straddle experts because every expert's segment in
// slot space is padded to a multiple of 128 rows.
//
// Reference counterpart: csrc/teramoe/teramoe_wrapper.cuh:46-98 (tile config), :530-780 (mainloop),
// csrc/teramoe/teramoe_sm100_bf16_compute.cuh:567-746 (SwiGLU epilogue).  Written from the PTX ISA
// description of tcgen05 / TMA, not from that code: different tile (128x256 vs 128x128), 8 epilogue
// warps, dSwiGLU and route-gradient fused in the epilogue, varlen-K weight-gradient mode.
#include "gemm.h"

#include <cuda.h>
#include <cuda_bf16.h>

#include "gemm_common.cuh"

namespace tmoe {

using namespace detail;

namespace {

// GATHER: 0 = operands are dense in slot space; 1 = operand A is gathered row-wise from a row source
// through gather_rows (TMA tile::gather4); 2 = operand B is gathered (weight-gradient mode only).
template <bool A_MN, bool B_MN, bool KGROUP, int EPI, int GATHER>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    // 128-byte swizzle needs 1024-byte aligned stage bases.
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + kStages * kStageBytes;
    // barrier words (8 bytes each): full[kStages], empty[kStages], tmem_full[2], tmem_empty[2]
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto tfull_bar = [&](int s) { return bar_base + 8u * (2 * kStages + s); };
    auto tempty_bar = [&](int s) { return bar_base + 8u * (2 * kStages + 2 + s); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + kStages * kStageBytes + 8 * (2 * kStages + 4));
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(tfull_bar(s), 1);
            mbar_init(tempty_bar(s), kEpiWarps);
        }
        fence_mbar_init();
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
    }
    if (warp == 2) tmem_alloc(smem_u32((const void*)tmem_slot), kTmemCols);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    int num_mblocks = g.max_mblocks;
    if constexpr (!KGROUP) {
        if (g.num_mblocks_dev != nullptr) num_mblocks = min(*g.num_mblocks_dev, g.max_mblocks);
    }

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (whole warp)
        // Lane 0 arms the barrier and issues the tiled loads; in the gather modes every lane issues the
        // gather4 copies of its own four rows, whose indices it keeps in registers.
        int stage = 0;
        uint32_t phase = 0;
        uint32_t issued = 0;
        bool ok = true;
        Tile tile;
        for (int t = blockIdx.x; ok && get_tile<KGROUP>(g, t, num_mblocks, tile); t += gridDim.x) {
            const int m0 = tile.m_blk * BM;
            const int n0 = tile.n_blk * BN;
            int4 ridx = make_int4(-1, -1, -1, -1);
            if constexpr (GATHER == 1 && !A_MN) ridx = *reinterpret_cast<const int4*>(g.gather_rows + m0 + 4 * lane);
            if constexpr (GATHER != 0 && KGROUP) {
                if (tile.nk > 0 && lane < 16) ridx = *reinterpret_cast<const int4*>(g.gather_rows + tile.k0 + 4 * lane);
            }
            for (int kb = 0; kb < tile.nk; ++kb) {
                int4 ridx_next = ridx;
                if constexpr (GATHER != 0 && KGROUP) {
                    if (kb + 1 < tile.nk && lane < 16)
                        ridx_next = *reinterpret_cast<const int4*>(g.gather_rows + tile.k0 + (kb + 1) * BK + 4 * lane);
                }
                if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, g.status, 100)) { ok = false; break; }
                const uint32_t a_dst = smem_base + stage * kStageBytes;
                const uint32_t b_dst = a_dst + kAStageBytes;
                const uint32_t bar = full_bar(stage);
                const int k = tile.k0 + kb * BK;
                if (lane == 0) {
                    mbar_arrive_expect_tx(bar, kStageBytes);
                    if constexpr (!A_MN) {
                        if constexpr (GATHER != 1) tma_load_2d(a_dst, &map_a, bar, k, m0);  // box {64 K, 128 rows}
                    } else if constexpr (GATHER != 1) {
#pragma unroll
                        for (int a = 0; a < BM / 64; ++a) tma_load_2d(a_dst + a * kAtomBytes, &map_a, bar, m0 + 64 * a, k);
                    }
                    if constexpr (!B_MN) {
                        tma_load_2d(b_dst, &map_b, bar, k, tile.group * g.b_group_rows + n0);  // box {64 K, 256 rows}
                    } else if constexpr (GATHER != 2) {
                        const int krow = KGROUP ? k : tile.group * g.b_group_rows + k;
#pragma unroll
                        for (int a = 0; a < BN / 64; ++a) tma_load_2d(b_dst + a * kAtomBytes, &map_b, bar, n0 + 64 * a, krow);
                    }
                }
                if constexpr (GATHER == 1 && !A_MN) {
                    // 128 rows x 64 K-columns: lane l owns rows 4l..4l+3 (512 bytes of the swizzled tile)
                    tma_gather4(a_dst + lane * 512, &map_a, bar, k, ridx);
                }
                if constexpr (GATHER == 1 && A_MN) {
                    // 64 K-rows per atom, gathered; lane l < 16 owns K-rows 4l..4l+3 of every 64-wide M atom
                    if (lane < 16) {
#pragma unroll
                        for (int a = 0; a < BM / 64; ++a) tma_gather4(a_dst + a * kAtomBytes + lane * 512, &map_a, bar, m0 + 64 * a, ridx);
                    }
                }
                if constexpr (GATHER == 2) {
                    if (lane < 16) {
#pragma unroll
                        for (int a = 0; a < BN / 64; ++a) tma_gather4(b_dst + a * kAtomBytes + lane * 512, &map_b, bar, n0 + 64 * a, ridx);
                    }
                }
                __syncwarp();
                ridx = (GATHER != 0 && KGROUP) ? ridx_next : ridx;
                ++issued;
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
        }
        if (!ok && lane == 0) {
            // Gave up: let copies that are still in flight land before the CTA's shared memory is released.
            const uint32_t pending = issued < (uint32_t)kStages ? issued : (uint32_t)kStages;
            for (uint32_t i = 0; i < pending; ++i) {
                const int s = (stage + kStages - 1 - (int)i) % kStages;
                const uint32_t ph = (s < stage) ? phase : (phase ^ 1u);
                const uint64_t t0 = globaltimer_ns();
                while (!mbar_try_wait(full_bar(s), ph) && globaltimer_ns() - t0 < 2000000ull) {}
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ UMMA issuer
        constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        Tile tile;
        int iter = 0;
        for (int t = blockIdx.x; ok && get_tile<KGROUP>(g, t, num_mblocks, tile); t += gridDim.x, ++iter) {
            const int as = iter & 1;
            const uint32_t aphase = (iter >> 1) & 1;
            if (!mbar_wait(tempty_bar(as), aphase ^ 1u, abort_flag, g.status, 200)) { ok = false; break; }
            tcgen05_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(as * BN);
            for (int kb = 0; kb < tile.nk; ++kb) {
                if (!mbar_wait(full_bar(stage), phase, abort_flag, g.status, 201)) { ok = false; break; }
                tcgen05_fence_after();
                if (elect_one()) {
                    const uint32_t a_addr = smem_base + stage * kStageBytes;
                    const uint32_t b_addr = a_addr + kAStageBytes;
#pragma unroll
                    for (int k = 0; k < BK / UK; ++k) {
                        // K-major: 32 bytes per UMMA_K inside the 128-byte swizzle row; 8-row groups 1024 B apart.
                        // MN-major: 16 K-rows of 128 B per UMMA_K; 64-wide MN atoms BK*128 B apart.
                        const uint64_t a_desc = A_MN ? make_smem_desc_sw128(a_addr + k * (UK * 128), kAtomBytes, 1024)
                                                     : make_smem_desc_sw128(a_addr + k * (UK * 2), 0, 1024);
                        const uint64_t b_desc = B_MN ? make_smem_desc_sw128(b_addr + k * (UK * 128), kAtomBytes, 1024)
                                                     : make_smem_desc_sw128(b_addr + k * (UK * 2), 0, 1024);
                        umma_bf16_ss(d_tmem, a_desc, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(empty_bar(stage));
                    if (kb == tile.nk - 1) umma_commit(tfull_bar(as));
                }
                __syncwarp();
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
            if (ok && tile.nk == 0) {
                if (elect_one()) umma_commit(tfull_bar(as));  // nothing to accumulate: epilogue writes zeros
                __syncwarp();
            }
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ epilogue
        const int q = warp & 3;          // TMEM lane quarter
        const int h = (warp - 4) >> 2;   // column half of the accumulator
        const int r = q * 32 + lane;     // row inside the tile
        bool ok = true;
        Tile tile;
        int iter = 0;
        for (int t = blockIdx.x; ok && get_tile<KGROUP>(g, t, num_mblocks, tile); t += gridDim.x, ++iter) {
            const int as = iter & 1;
            const uint32_t aphase = (iter >> 1) & 1;
            if (!mbar_wait(tfull_bar(as), aphase, abort_flag, g.status, 300)) { ok = false; break; }
            tcgen05_fence_after();
            const uint32_t taddr0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(as * BN + h * (BN / 2));
            const int n0 = tile.n_blk * BN + h * (BN / 2);  // first accumulator column handled by this thread
            const bool zero_tile = (tile.nk == 0);
            long row;
            bool row_ok = true;
            if constexpr (!KGROUP) {
                row = (long)tile.m_blk * BM + r;
            } else {
                row_ok = (tile.m_blk * BM + r) < g.m_total;
                row = (long)tile.group * g.m_total + tile.m_blk * BM + r;
            }
            epilogue_thread<EPI>(g, taddr0, row, row_ok, n0, tile.n_blk * 2 + h, zero_tile);
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(as));
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 2) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
template <bool A_MN, bool B_MN, bool KGROUP, int EPI, int GATHER>
cudaError_t launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& g, int total_tiles, int num_sms,
                   cudaStream_t stream) {
    auto kern = grouped_gemm_kernel<A_MN, B_MN, KGROUP, EPI, GATHER>;
    static bool configured[64] = {};
    if (cudaError_t e = ensure_smem_limit(kern, kSmemBytes, configured); e != cudaSuccess) return e;
    if (total_tiles <= 0) return cudaSuccess;
    int grid = total_tiles < num_sms ? total_tiles : num_sms;
    kern<<<grid, kThreads, kSmemBytes, stream>>>(ma, mb, g);
    return cudaGetLastError();
}

// The TMA tile::gather4 operand modes measured about three times slower than a dense slot-space operand, so their
// kernels are only compiled when the library is built with -DTMOE_WITH_GATHER4; otherwise asking for them is an error.
#ifdef TMOE_WITH_GATHER4
#define TMOE_GATHER_LAUNCH(call) call
#else
#define TMOE_GATHER_LAUNCH(call) cudaErrorNotSupported
#endif

void set_push(GemmArgs& g, const PushTarget& p) {
    g.push_ptrs = reinterpret_cast<const unsigned long long*>(p.arena_ptrs);
    g.push_off = p.landing_off;
    g.slot_tk = p.slot_tk;
    g.slot_row = p.slot_row;
    g.recv_row_base = p.recv_row_base;
    g.num_ranks = p.num_ranks;
}

}  // namespace

int gemm_num_droute_parts(int I) { return 2 * ((I + BN - 1) / BN); }

cudaError_t gemm_fwd_gateup(const void* xperm, const void* w_gateup, void* act, void* preact, const float* row_w,
                            const MGroupLayout& lay, int H, int I, int num_local_experts, const int* gather_rows, int src_rows, int* status, int num_sms,
                            cudaStream_t stream) {
    const int max_mblocks = lay.max_mblocks;
    if (max_mblocks <= 0) return cudaSuccess;
    if (H % BK != 0 || I % 32 != 0) return cudaErrorInvalidValue;
    CUtensorMap ma, mb;
    cudaError_t e;
    if (gather_rows != nullptr) {
        if ((e = make_map(&ma, xperm, (uint64_t)(src_rows > 0 ? src_rows : 1), H, BK, 1)) != cudaSuccess) return e;
    } else {
        if ((e = make_map(&ma, xperm, (uint64_t)max_mblocks * BM, H, BK, BM)) != cudaSuccess) return e;
    }
    if ((e = make_map(&mb, w_gateup, (uint64_t)num_local_experts * 2 * I, H, BK, BN)) != cudaSuccess) return e;
    GemmArgs g{};
    g.n_total = 2 * I;
    g.k_total = H;
    g.num_n_blocks = (2 * I + BN - 1) / BN;
    g.max_mblocks = max_mblocks;
    g.num_mblocks_dev = lay.num_mblocks_dev;
    g.mblock_expert = lay.mblock_expert;
    g.unit_blk = lay.unit_blk;
    g.num_units_dev = lay.num_units_dev;
    g.max_units = lay.max_units;
    g.b_group_rows = 2 * I;
    g.d = static_cast<__nv_bfloat16*>(act);
    g.ldd = I;
    g.aux = static_cast<__nv_bfloat16*>(preact);
    g.ld_aux = 2 * I;
    g.row_w = row_w;
    g.status = status;
    g.gather_rows = gather_rows;
    if (lay.unit_blk != nullptr && gather_rows == nullptr)
        return gemm2_mgroup(0, xperm, w_gateup, g, max_mblocks * BM, H, num_local_experts * 2 * I, H, num_sms, stream);
    if (gather_rows != nullptr)
        return TMOE_GATHER_LAUNCH((launch<false, false, false, kEpiSwiGLU, 1>(ma, mb, g, max_mblocks * g.num_n_blocks, default_sms(num_sms), stream)));
    return launch<false, false, false, kEpiSwiGLU, 0>(ma, mb, g, max_mblocks * g.num_n_blocks, default_sms(num_sms), stream);
}

cudaError_t gemm_fwd_down(const void* act, const void* w_down, void* y, const MGroupLayout& lay, int H, int I,
                          int num_local_experts, int* status, int num_sms, cudaStream_t stream, const PushTarget* push) {
    const int max_mblocks = lay.max_mblocks;
    if (max_mblocks <= 0) return cudaSuccess;
    if (I % BK != 0 || H % 8 != 0) return cudaErrorInvalidValue;
    CUtensorMap ma, mb;
    cudaError_t e;
    if ((e = make_map(&ma, act, (uint64_t)max_mblocks * BM, I, BK, BM)) != cudaSuccess) return e;
    if ((e = make_map(&mb, w_down, (uint64_t)num_local_experts * H, I, BK, BN)) != cudaSuccess) return e;
    GemmArgs g{};
    g.n_total = H;
    g.k_total = I;
    g.num_n_blocks = (H + BN - 1) / BN;
    g.max_mblocks = max_mblocks;
    g.num_mblocks_dev = lay.num_mblocks_dev;
    g.mblock_expert = lay.mblock_expert;
    g.unit_blk = lay.unit_blk;
    g.num_units_dev = lay.num_units_dev;
    g.max_units = lay.max_units;
    g.b_group_rows = H;
    g.d = static_cast<__nv_bfloat16*>(y);
    g.ldd = H;
    g.status = status;
    if (push != nullptr) {
        set_push(g, *push);
        if (lay.unit_blk != nullptr) return gemm2_mgroup(4, act, w_down, g, max_mblocks * BM, I, num_local_experts * H, I, num_sms, stream);
        return launch<false, false, false, kEpiPush, 0>(ma, mb, g, max_mblocks * g.num_n_blocks, default_sms(num_sms), stream);
    }
    if (lay.unit_blk != nullptr) return gemm2_mgroup(1, act, w_down, g, max_mblocks * BM, I, num_local_experts * H, I, num_sms, stream);
    return launch<false, false, false, kEpiStore, 0>(ma, mb, g, max_mblocks * g.num_n_blocks, default_sms(num_sms), stream);
}

cudaError_t gemm_bwd_gradact(const void* dyperm, const void* w_down, const void* preact, const float* row_w, void* dgu,
                             void* act_w, float* droute_part, const MGroupLayout& lay, int H, int I, int num_local_experts, const int* gather_rows, int src_rows,
                             int* status, int num_sms, cudaStream_t stream) {
    const int max_mblocks = lay.max_mblocks;
    if (max_mblocks <= 0) return cudaSuccess;
    if (H % BK != 0 || I % 32 != 0) return cudaErrorInvalidValue;
    CUtensorMap ma, mb;
    cudaError_t e;
    if (gather_rows != nullptr) {
        if ((e = make_map(&ma, dyperm, (uint64_t)(src_rows > 0 ? src_rows : 1), H, BK, 1)) != cudaSuccess) return e;
    } else {
        if ((e = make_map(&ma, dyperm, (uint64_t)max_mblocks * BM, H, BK, BM)) != cudaSuccess) return e;
    }
    // W_down [E*H, I]: K = H rows, N = I contiguous -> MN-major B, box {64 N, 64 K}
    if ((e = make_map(&mb, w_down, (uint64_t)num_local_experts * H, I, 64, BK)) != cudaSuccess) return e;
    GemmArgs g{};
    g.n_total = I;
    g.k_total = H;
    g.num_n_blocks = (I + BN - 1) / BN;
    g.max_mblocks = max_mblocks;
    g.num_mblocks_dev = lay.num_mblocks_dev;
    g.mblock_expert = lay.mblock_expert;
    g.unit_blk = lay.unit_blk;
    g.num_units_dev = lay.num_units_dev;
    g.max_units = lay.max_units;
    g.b_group_rows = H;
    g.d = static_cast<__nv_bfloat16*>(act_w);
    g.ldd = I;
    g.aux = static_cast<__nv_bfloat16*>(dgu);
    g.ld_aux = 2 * I;
    g.preact = static_cast<const __nv_bfloat16*>(preact);
    g.row_w = row_w;
    g.droute_part = droute_part;
    g.n_parts = gemm_num_droute_parts(I);
    g.status = status;
    g.gather_rows = gather_rows;
    if (lay.unit_blk != nullptr && gather_rows == nullptr)
        return gemm2_mgroup(2, dyperm, w_down, g, max_mblocks * BM, H, num_local_experts * H, I, num_sms, stream);
    if (gather_rows != nullptr)
        return TMOE_GATHER_LAUNCH((launch<false, true, false, kEpiDSwiGLU, 1>(ma, mb, g, max_mblocks * g.num_n_blocks, default_sms(num_sms), stream)));
    return launch<false, true, false, kEpiDSwiGLU, 0>(ma, mb, g, max_mblocks * g.num_n_blocks, default_sms(num_sms), stream);
}

cudaError_t gemm_bwd_dx(const void* dgu, const void* w_gateup, void* dxperm, const MGroupLayout& lay, int H, int I,
                        int num_local_experts, int* status, int num_sms, cudaStream_t stream, const PushTarget* push) {
    const int max_mblocks = lay.max_mblocks;
    if (max_mblocks <= 0) return cudaSuccess;
    if ((2 * I) % BK != 0 || H % 8 != 0) return cudaErrorInvalidValue;
    CUtensorMap ma, mb;
    cudaError_t e;
    if ((e = make_map(&ma, dgu, (uint64_t)max_mblocks * BM, 2 * I, BK, BM)) != cudaSuccess) return e;
    // W_gateup [E*2I, H]: K = 2I rows, N = H contiguous -> MN-major B
    if ((e = make_map(&mb, w_gateup, (uint64_t)num_local_experts * 2 * I, H, 64, BK)) != cudaSuccess) return e;
    GemmArgs g{};
    g.n_total = H;
    g.k_total = 2 * I;
    g.num_n_blocks = (H + BN - 1) / BN;
    g.max_mblocks = max_mblocks;
    g.num_mblocks_dev = lay.num_mblocks_dev;
    g.mblock_expert = lay.mblock_expert;
    g.unit_blk = lay.unit_blk;
    g.num_units_dev = lay.num_units_dev;
    g.max_units = lay.max_units;
    g.b_group_rows = 2 * I;
    g.d = static_cast<__nv_bfloat16*>(dxperm);
    g.ldd = H;
    g.status = status;
    if (push != nullptr) {
        set_push(g, *push);
        if (lay.unit_blk != nullptr)
            return gemm2_mgroup(5, dgu, w_gateup, g, max_mblocks * BM, 2 * I, num_local_experts * 2 * I, H, num_sms, stream);
        return launch<false, true, false, kEpiPush, 0>(ma, mb, g, max_mblocks * g.num_n_blocks, default_sms(num_sms), stream);
    }
    if (lay.unit_blk != nullptr)
        return gemm2_mgroup(3, dgu, w_gateup, g, max_mblocks * BM, 2 * I, num_local_experts * 2 * I, H, num_sms, stream);
    return launch<false, true, false, kEpiStore, 0>(ma, mb, g, max_mblocks * g.num_n_blocks, default_sms(num_sms), stream);
}

cudaError_t gemm_wgrad(const void* a, const void* b, void* dw, const int* seg_offsets, int total_rows, int M, int N,
                       int num_local_experts, const int* gather_rows, int gather_operand, int src_rows, bool cta_pairs, int* status,
                       int num_sms, cudaStream_t stream) {
    if (num_local_experts <= 0) return cudaSuccess;
    if (M % 8 != 0 || N % 8 != 0) return cudaErrorInvalidValue;
    // The tensor maps must cover at least one row so that encoding succeeds when nothing was received.
    const uint64_t rows = total_rows > 0 ? (uint64_t)total_rows : 1;
    CUtensorMap ma, mb;
    cudaError_t e;
    const uint64_t srows = src_rows > 0 ? (uint64_t)src_rows : 1;
    if (gather_rows == nullptr) gather_operand = 0;
    if ((e = gather_operand == 1 ? make_map(&ma, a, srows, M, 64, 1) : make_map(&ma, a, rows, M, 64, BK)) != cudaSuccess) return e;
    if ((e = gather_operand == 2 ? make_map(&mb, b, srows, N, 64, 1) : make_map(&mb, b, rows, N, 64, BK)) != cudaSuccess) return e;
    GemmArgs g{};
    g.n_total = N;
    g.num_n_blocks = (N + BN - 1) / BN;
    g.max_mblocks = (M + BM - 1) / BM;
    g.num_groups = num_local_experts;
    g.seg_offsets = seg_offsets;
    g.m_total = M;
    g.d = static_cast<__nv_bfloat16*>(dw);
    g.ldd = N;
    g.status = status;
    g.gather_rows = gather_rows;
    const int tiles = num_local_experts * g.max_mblocks * g.num_n_blocks;
    if (cta_pairs && gather_operand == 0 && total_rows > 0) return gemm2_wgrad(a, b, g, total_rows, M, N, num_sms, stream);
    if (gather_operand == 1) return TMOE_GATHER_LAUNCH((launch<true, true, true, kEpiStore, 1>(ma, mb, g, tiles, default_sms(num_sms), stream)));
    if (gather_operand == 2) return TMOE_GATHER_LAUNCH((launch<true, true, true, kEpiStore, 2>(ma, mb, g, tiles, default_sms(num_sms), stream)));
    return launch<true, true, true, kEpiStore, 0>(ma, mb, g, tiles, default_sms(num_sms), stream);
}

bool gemm_has_gather4() {
#ifdef TMOE_WITH_GATHER4
    return true;
#else
    return false;
#endif
}

}  // namespace tmoe
