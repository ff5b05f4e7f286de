// CTA-pair variant of the grouped GEMM family: thread-block clusters of two CTAs on neighbouring SMs
// compute one 256 x 256 tile with tcgen05 cta_group::2.
//
// Each CTA of the pair loads its own 128 rows of A and HALF of the B tile (128 of the 256 N columns);
// the UMMA, issued by one thread of the pair's first CTA, reads both CTAs' shared memory and writes
// both CTAs' tensor memory (128 accumulator rows each).  Per CTA a pipeline stage is 32 KB instead
// of 48 KB, so six stages fit and the L2 -> SM traffic per FLOP drops by a third.
//
// Measured on B200 (H=7168, I=2048, 32 experts x 2048 rows): 1437 / 1523 / 1373 / 1545 TFLOP/s for
// gate_up / down / grad_act / dX and 1259 / 1268 for the two weight gradients, against 1359 / 1297 /
// 1171 / 1396 / 987 / 1004 for the one-CTA kernels; results are bitwise identical.  Remote mbarrier
// arrives must use CTA-scope release (ptx.cuh mbar_arrive_cluster): with a cluster-scope release
// every arrive paid a fence and the same kernels ran at 600-780 TFLOP/s.  Every CTA loads
// its operands itself with plain (non-multicast) TMA loads from local memory; only barrier arrivals
// cross the pair (tcgen05.commit to both CTAs, remote mbarrier arrives).
//
// M-grouped modes work on "units": one or two consecutive 128-row blocks of the same expert.  A unit
// with a single block (experts with an odd block count) still occupies the pair; the second CTA's
// rows are ignored.  The weight-gradient mode pairs along the weight rows.
//
// Reference counterpart: the optional MK_COMPUTE_KERNEL=2 path (csrc/teramoe/teramoe_wrapper.cuh:77-79,
// :569, :655-659), which is not the reference's default.
#include <cstdlib>

#include "gemm.h"
#include "gemm_common.cuh"

namespace tmoe {

using namespace detail;

namespace {

// Pipeline depth: six 32 KB stages; the push epilogue gives one stage up for its staging buffers.
__host__ __device__ constexpr int stages_for(int epi) { return epi == kEpiPush ? 5 : 6; }
__host__ __device__ constexpr int smem_bytes_for(int epi) {
    return stages_for(epi) * (16384 + 16384) + 1024 + 256 + (epi == kEpiPush ? kEpiWarps * kPushWarpBytes : 0);
}
constexpr int kBHalfBytes = (BN / 2) * BK * 2;                 // 16 KB: this CTA's half of the B tile
constexpr int kStageBytes2 = kAStageBytes + kBHalfBytes;       // 32 KB

constexpr int kSuperU = 8;                                      // units per L2 super-group

struct Tile2 {
    int blk0, two, n_blk, group, k0, nk, m_unit;
};

template <bool KGROUP>
__device__ __forceinline__ bool get_tile2(const GemmArgs& g, int t, int num_units, Tile2& tile) {
    if constexpr (!KGROUP) {
        const int total = num_units * g.num_n_blocks;
        if (t >= total) return false;
        const int per_super = kSuperU * g.num_n_blocks;
        const int super = t / per_super;
        const int r = t - super * per_super;
        const int u_first = super * kSuperU;
        const int u_cnt = min(kSuperU, num_units - u_first);
        tile.n_blk = r / u_cnt;
        const int u = u_first + (r - tile.n_blk * u_cnt);
        tile.blk0 = g.unit_blk[u];
        tile.two = (g.unit_blk[u + 1] - tile.blk0) == 2;
        tile.group = g.mblock_expert[tile.blk0];
        tile.k0 = 0;
        tile.nk = g.k_total / BK;
        tile.m_unit = u;
        return true;
    } else {
        const int m_units = (g.m_total + 2 * BM - 1) / (2 * BM);
        const int per_group = m_units * g.num_n_blocks;
        const int total = g.num_groups * per_group;
        if (t >= total) return false;
        tile.group = t / per_group;
        const int r = t - tile.group * per_group;
        if (g.kgroup_n_fast) {
            tile.m_unit = r / g.num_n_blocks;
            tile.n_blk = r - tile.m_unit * g.num_n_blocks;
        } else {
            tile.n_blk = r / m_units;
            tile.m_unit = r - tile.n_blk * m_units;
        }
        tile.blk0 = 0;
        tile.two = 1;
        const int s0 = g.seg_offsets[tile.group];
        const int s1 = g.seg_offsets[tile.group + 1];
        tile.k0 = s0;
        tile.nk = (s1 - s0) / BK;
        return true;
    }
}

template <bool A_MN, bool B_MN, bool KGROUP, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
grouped_gemm2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const __grid_constant__ GemmArgs g) {
    constexpr int kStages2 = stages_for(EPI);
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + kStages2 * kStageBytes2;
    const uint32_t push_stage_base = bar_base + 256;           // kEpiPush: staging rows of the epilogue warps
    auto full_bar = [&](int s) { return bar_base + 8u * s; };                       // used in CTA 0 only
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages2 + s); };          // one per CTA
    auto tfull_bar = [&](int s) { return bar_base + 8u * (2 * kStages2 + s); };      // one per CTA
    auto tempty_bar = [&](int s) { return bar_base + 8u * (2 * kStages2 + 2 + s); }; // used in CTA 0 only
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + kStages2 * kStageBytes2 + 8 * (2 * kStages2 + 4));
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int cluster_id = blockIdx.x >> 1;
    const int num_clusters = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        for (int s = 0; s < kStages2; ++s) {
            mbar_init(full_bar(s), 2);            // one arrive per CTA's producer
            mbar_init(empty_bar(s), 1);           // tcgen05.commit of the pair's UMMA thread
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(tfull_bar(s), 1);
            mbar_init(tempty_bar(s), 2 * kEpiWarps);  // epilogue warps of both CTAs
        }
        fence_mbar_init();
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
    }
    if (warp == 2) tmem_alloc_2cta(smem_u32((const void*)tmem_slot), kTmemCols);
    tcgen05_fence_before();
    cluster_sync_all();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    int num_units = g.max_units;
    if constexpr (!KGROUP) {
        if (g.num_units_dev != nullptr) num_units = min(*g.num_units_dev, g.max_units);
    }

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            Tile2 tile;
            for (int t = cluster_id; ok && get_tile2<KGROUP>(g, t, num_units, tile); t += num_clusters) {
                const int m0 = KGROUP ? (tile.m_unit * 2 + (int)rank) * BM : (tile.blk0 + (int)rank) * BM;
                const int n0 = tile.n_blk * BN + (int)rank * (BN / 2);   // this CTA's half of the N columns
                for (int kb = 0; kb < tile.nk; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, g.status, 110)) { ok = false; break; }
                    const uint32_t a_dst = smem_base + stage * kStageBytes2;
                    const uint32_t b_dst = a_dst + kAStageBytes;
                    const uint32_t bar = mapa_shared(full_bar(stage), 0);   // the pair's barrier lives in CTA 0
                    if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * kStageBytes2);
                    else mbar_arrive_cluster(bar);
                    const int k = tile.k0 + kb * BK;
                    if constexpr (!A_MN) {
                        tma_load_2d_2cta(a_dst, &map_a, bar, k, m0);
                    } else {
#pragma unroll
                        for (int a = 0; a < BM / 64; ++a) tma_load_2d_2cta(a_dst + a * kAtomBytes, &map_a, bar, m0 + 64 * a, k);
                    }
                    if constexpr (!B_MN) {
                        tma_load_2d_2cta(b_dst, &map_b, bar, k, tile.group * g.b_group_rows + n0);   // box {64 K, 128 rows}
                    } else {
                        const int krow = KGROUP ? k : tile.group * g.b_group_rows + k;
#pragma unroll
                        for (int a = 0; a < BN / 128; ++a) tma_load_2d_2cta(b_dst + a * kAtomBytes, &map_b, bar, n0 + 64 * a, krow);
                    }
                    if (++stage == kStages2) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1 && rank == 0) {
        // ------------------------------------------------------------------ UMMA issuer (first CTA of the pair)
        constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN, B_MN);
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        Tile2 tile;
        int iter = 0;
        for (int t = cluster_id; ok && get_tile2<KGROUP>(g, t, num_units, tile); t += num_clusters, ++iter) {
            const int as = iter & 1;
            const uint32_t aphase = (iter >> 1) & 1;
            if (!mbar_wait(tempty_bar(as), aphase ^ 1u, abort_flag, g.status, 210)) { ok = false; break; }
            tcgen05_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(as * BN);
            for (int kb = 0; kb < tile.nk; ++kb) {
                if (!mbar_wait(full_bar(stage), phase, abort_flag, g.status, 211)) { ok = false; break; }
                tcgen05_fence_after();
                if (elect_one()) {
                    const uint32_t a_addr = smem_base + stage * kStageBytes2;
                    const uint32_t b_addr = a_addr + kAStageBytes;
#pragma unroll
                    for (int k = 0; k < BK / UK; ++k) {
                        const uint64_t a_desc = A_MN ? make_smem_desc_sw128(a_addr + k * (UK * 128), kAtomBytes, 1024)
                                                     : make_smem_desc_sw128(a_addr + k * (UK * 2), 0, 1024);
                        const uint64_t b_desc = B_MN ? make_smem_desc_sw128(b_addr + k * (UK * 128), kAtomBytes, 1024)
                                                     : make_smem_desc_sw128(b_addr + k * (UK * 2), 0, 1024);
                        umma_bf16_ss_2cta(d_tmem, a_desc, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit_2cta(empty_bar(stage), 3u);
                    if (kb == tile.nk - 1) umma_commit_2cta(tfull_bar(as), 3u);
                }
                __syncwarp();
                if (++stage == kStages2) { stage = 0; phase ^= 1u; }
            }
            if (ok && tile.nk == 0) {
                if (elect_one()) umma_commit_2cta(tfull_bar(as), 3u);
                __syncwarp();
            }
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
        const int q = warp & 3;
        const int h = (warp - 4) >> 2;
        const int r = q * 32 + lane;
        bool ok = true;
        Tile2 tile;
        int iter = 0;
        for (int t = cluster_id; ok && get_tile2<KGROUP>(g, t, num_units, tile); t += num_clusters, ++iter) {
            const int as = iter & 1;
            const uint32_t aphase = (iter >> 1) & 1;
            if (!mbar_wait(tfull_bar(as), aphase, abort_flag, g.status, 310)) { ok = false; break; }
            tcgen05_fence_after();
            const uint32_t taddr0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(as * BN + h * (BN / 2));
            const int n0 = tile.n_blk * BN + h * (BN / 2);
            long row;
            bool row_ok, live;
            if constexpr (!KGROUP) {
                live = (rank == 0) || tile.two;
                row_ok = live;
                row = (long)(tile.blk0 + (int)rank) * BM + r;
            } else {
                const int m = (tile.m_unit * 2 + (int)rank) * BM + r;
                live = true;
                row_ok = m < g.m_total;
                row = (long)tile.group * g.m_total + m;
            }
            if constexpr (EPI == kEpiPush) {
                const unsigned long long dst_row = push_row_address(g, row, live, nullptr);
                const uint32_t my_row_smem = push_stage_base + (uint32_t)(warp - 4) * kPushWarpBytes + (uint32_t)lane * kPushRowBytes;
                push_epilogue_warp(g, taddr0, dst_row, n0, my_row_smem);
            } else {
                if (live) epilogue_thread<EPI>(g, taddr0, row_ok ? row : 0, row_ok, n0, tile.n_blk * 2 + h, tile.nk == 0);
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_shared(tempty_bar(as), 0));
        }
        if constexpr (EPI == kEpiPush) tma_store_wait<0>();   // every pushed segment of this lane has been written
    }

    tcgen05_fence_before();
    cluster_sync_all();
    if (warp == 2) {
        tcgen05_fence_after();
        tmem_dealloc_2cta(tmem_base, kTmemCols);
    }
}

template <bool A_MN, bool B_MN, bool KGROUP, int EPI>
cudaError_t launch2(const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& g, int total_tiles, int num_sms, cudaStream_t stream) {
    auto kern = grouped_gemm2_kernel<A_MN, B_MN, KGROUP, EPI>;
    constexpr int kSmemBytes2 = smem_bytes_for(EPI);
    static bool configured[64] = {};
    if (cudaError_t e = ensure_smem_limit(kern, kSmemBytes2, configured); e != cudaSuccess) return e;
    if (total_tiles <= 0) return cudaSuccess;
    int grid = 2 * total_tiles < num_sms ? 2 * total_tiles : num_sms;
    grid &= ~1;
    if (grid < 2) grid = 2;
    kern<<<grid, kThreads, kSmemBytes2, stream>>>(ma, mb, g);
    return cudaGetLastError();
}

}  // namespace

cudaError_t gemm2_mgroup(int kind, const void* a, const void* b, const GemmArgs& g_in, int a_rows, int a_cols, int b_rows, int b_cols,
                         int num_sms, cudaStream_t stream) {
    // kind: 0 gate_up+SwiGLU, 1 down, 2 grad_act+dSwiGLU, 3 dX, 4 down with pushed rows, 5 dX with pushed rows
    GemmArgs g = g_in;
    CUtensorMap ma, mb;
    cudaError_t e;
    if ((e = make_map(&ma, a, (uint64_t)a_rows, a_cols, BK, BM)) != cudaSuccess) return e;
    const bool b_mn = (kind == 2 || kind == 3 || kind == 5);
    if ((e = b_mn ? make_map(&mb, b, (uint64_t)b_rows, b_cols, 64, BK) : make_map(&mb, b, (uint64_t)b_rows, b_cols, BK, BN / 2)) != cudaSuccess)
        return e;
    const int tiles = g.max_units * g.num_n_blocks;
    const int sms = default_sms(num_sms);
    // the push epilogue hands whole 128-byte segments (64 columns) to bulk copies: 16-byte aligned rows, no ragged edge
    if ((kind == 4 || kind == 5) && (g.n_total % 64 != 0 || g.ldd % 8 != 0 || g.push_off % 16 != 0)) return cudaErrorInvalidValue;
    switch (kind) {
        case 0: return launch2<false, false, false, kEpiSwiGLU>(ma, mb, g, tiles, sms, stream);
        case 1: return launch2<false, false, false, kEpiStore>(ma, mb, g, tiles, sms, stream);
        case 2: return launch2<false, true, false, kEpiDSwiGLU>(ma, mb, g, tiles, sms, stream);
        case 4: return launch2<false, false, false, kEpiPush>(ma, mb, g, tiles, sms, stream);
        case 5: return launch2<false, true, false, kEpiPush>(ma, mb, g, tiles, sms, stream);
        default: return launch2<false, true, false, kEpiStore>(ma, mb, g, tiles, sms, stream);
    }
}

cudaError_t gemm2_wgrad(const void* a, const void* b, const GemmArgs& g_in, int rows, int M, int N, int num_sms, cudaStream_t stream) {
    GemmArgs g = g_in;
    {
        // experiment switch: TMOE_WGRAD_ORDER=n / m forces the order in which consecutive tiles walk dW; default: row units first
        static const char* env = getenv("TMOE_WGRAD_ORDER");
        g.kgroup_n_fast = (env != nullptr && env[0] == 'n') ? 1 : 0;
    }
    CUtensorMap ma, mb;
    cudaError_t e;
    if ((e = make_map(&ma, a, (uint64_t)rows, M, 64, BK)) != cudaSuccess) return e;
    if ((e = make_map(&mb, b, (uint64_t)rows, N, 64, BK)) != cudaSuccess) return e;
    const int m_units = (M + 2 * BM - 1) / (2 * BM);
    return launch2<true, true, true, kEpiStore>(ma, mb, g, g.num_groups * m_units * g.num_n_blocks, default_sms(num_sms), stream);
}

}  // namespace tmoe
