// Fused dispatch + grouped GEMM: ONE cooperative kernel in which a few CTA pairs push this rank's
// routed rows straight into the peers' slot-space operand buffers over NVLink while all other CTA
// pairs run the tcgen05 (cta_group::2) GEMM that consumes the rows arriving from the peers.
//
//   dispatch pairs   walk this rank's (token,k) entries in sending order (own rank first, then rank+1,
//                    ... so that at any moment every rank receives from one sender), copy each row
//                    into slot `send_slot` of the destination's operand buffer (bulk copies staged in
//                    shared memory, one row in flight per warp) and then publish it: bulk-group wait,
//                    fence.acq_rel.sys + red.add on the destination's per-block arrival counter.
//                    In forward they also store the slot tables (route weight, entry id, row).
//                    When its rows are out, a dispatch pair joins the compute pairs.
//   compute pairs    the CTA-pair GEMM of gemm2.cu over the tiles in arrival order (arrival_order in routing.cu).
//                    Tiles are claimed from one counter per launch (atomicAdd by the first CTA's producer thread,
//                    one tile ahead) and handed to the other roles of the pair through a 4-entry ring in each
//                    CTA's shared memory.  Before the first load of a tile the producer thread waits (bounded,
//                    ld.acquire.sys) until the arrival counter of its 128-row block has reached the block's row
//                    count, then fence.proxy.async, then TMA.  Weights never wait.
//
// Forward:  GU = Xslots . Wgu^T with the SwiGLU x route epilogue (pre-activation side store).
// Backward: gA = dYslots . Wd with the dSwiGLU epilogue (dGU, act x route, route-gradient partials).
//
// Reference counterpart: the dispatch + compute roles of teramoe_fused_forward_kernel /
// teramoe_fused_backward_kernel (csrc/teramoe/teramoe_orchestrator.cu:524-1369, :1626-1907, :2978-3042,
// :4495-4848).  Differences: rows go to their final slot (no receive ring, no publisher warps), there is no
// scheduler SM (tiles are claimed from a counter in the arrival order computed by arrival_order in routing.cu),
// readiness is one counter per 128-row block, dispatch SMs are reused for compute, and every wait is bounded.
#include "fused.h"

#include "gemm_common.cuh"

namespace tmoe {

using namespace detail;

namespace {

constexpr int kStagesF = 6;
constexpr int kBHalfBytesF = (BN / 2) * BK * 2;
constexpr int kStageBytesF = kAStageBytes + kBHalfBytesF;       // 32 KB
constexpr int kSmemBytesF = kStagesF * kStageBytesF + 1024 + 512;
constexpr int kSuperUF = 8;
constexpr int kDispatchChunk = 8192;                            // two per dispatch warp; 12 warps fill the six operand stages
constexpr int kPublishBatch = 4;                                // rows published per system-scope fence
constexpr int kSchedDepth = 4;                                  // entries of the tile ring (the producer runs < 4 tiles ahead of the epilogue)
constexpr uint32_t kSchedFullOffset = 336, kSchedEmptyOffset = 368, kRingOffset = 400;   // bytes after the pipeline barriers
// arrivals that release a ring entry: UMMA issuer + 8 epilogue warps of the first CTA, producer + 8 epilogue warps of the second
constexpr uint32_t kSchedConsumers = 2 * kEpiWarps + 2;
static_assert((kThreads / 32) * 2 * kDispatchChunk <= kStagesF * kStageBytesF, "dispatch staging exceeds the operand stages");

struct TileF {
    int blk0, two, n_blk, group;
};

__device__ __forceinline__ bool get_tile_f(const GemmArgs& g, const int* unit_order, int t, int t_end, int num_units, TileF& tile) {
    if (t >= t_end) return false;
    const int per_super = kSuperUF * g.num_n_blocks;
    const int super = t / per_super;
    const int r = t - super * per_super;
    const int u_first = super * kSuperUF;
    const int u_cnt = min(kSuperUF, num_units - u_first);
    tile.n_blk = r / u_cnt;
    const int u = unit_order[u_first + (r - tile.n_blk * u_cnt)];
    tile.blk0 = g.unit_blk[u];
    tile.two = (g.unit_blk[u + 1] - tile.blk0) == 2;
    tile.group = g.mblock_expert[tile.blk0];
    return true;
}

__device__ __forceinline__ long long load_idx(const void* idx, int is64, long i) {
    return is64 ? reinterpret_cast<const long long*>(idx)[i] : (long long) reinterpret_cast<const int*>(idx)[i];
}

__device__ __forceinline__ void red_add_relaxed_sys(int* p, int v) {
    asm volatile("red.relaxed.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <bool B_MN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
fused_dispatch_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                           const __grid_constant__ GemmArgs g, const __grid_constant__ FusedArgs f) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + kStagesF * kStageBytesF;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStagesF + s); };
    auto tfull_bar = [&](int s) { return bar_base + 8u * (2 * kStagesF + s); };
    auto tempty_bar = [&](int s) { return bar_base + 8u * (2 * kStagesF + 2 + s); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + kStagesF * kStageBytesF + 8 * (2 * kStagesF + 4));
    volatile uint32_t* abort_flag = tmem_slot + 1;
    auto dispatch_bar = [&](int w, uint32_t b) { return bar_base + 144u + 8u * (2u * w + b); };   // two per dispatch warp, after the flags

    auto sched_full = [&](int e) { return bar_base + kSchedFullOffset + 8u * e; };
    auto sched_empty = [&](int e) { return bar_base + kSchedEmptyOffset + 8u * e; };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int cluster_id = blockIdx.x >> 1;
    const int num_clusters = gridDim.x >> 1;
    const int cd = f.num_dispatch_clusters;
    const bool is_dispatch = cluster_id < cd;

    // Every CTA sets its barriers and tensor memory up the same way (tcgen05 alloc is collective over the pair).
    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        for (int s = 0; s < kStagesF; ++s) {
            mbar_init(full_bar(s), 2);
            mbar_init(empty_bar(s), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(tfull_bar(s), 1);
            mbar_init(tempty_bar(s), 2 * kEpiWarps);
        }
        for (int w = 0; w < kThreads / 32; ++w) {
            mbar_init(dispatch_bar(w, 0), 1);
            mbar_init(dispatch_bar(w, 1), 1);
        }
        for (int e = 0; e < kSchedDepth; ++e) {
            mbar_init(sched_full(e), 1);
            mbar_init(sched_empty(e), kSchedConsumers);
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

    if (is_dispatch) {
        // ------------------------------------------------------------------ dispatch role (all 12 warps)
        // Each warp owns two 8 KB staging buffers in the (otherwise unused) operand stages.  Its leader streams
        // the rows through them in chunks with bulk copies: global -> shared (completes on the buffer's
        // mbarrier), shared -> the destination's slot row (bulk group); the load of chunk c runs while chunk
        // c-1 is stored.  Rows are published in batches (arrival counter of the row's 128-row block at the
        // destination): bulk-group wait, one system-scope fence, one red.add per row.
        const int num_send = min(*f.num_send, f.max_send);
        const int warps_total = cd * 2 * (kThreads / 32);
        const int wid = (cluster_id * 2 + (int)rank) * (kThreads / 32) + warp;
        const int e_local = f.E / f.N;
        if (lane == 0) {
            const uint32_t buf0 = smem_base + (uint32_t)warp * (2 * kDispatchChunk);
            const uint32_t row_bytes = (uint32_t)f.H * 2u;
            uint32_t ph0 = 0, ph1 = 0, nchunk = 0;
            bool ok = true;
            // chunk whose load is in flight (stored one step later)
            bool pend = false, pend_last = false;
            uint64_t pend_dst = 0;
            uint32_t pend_bytes = 0, pend_b = 0;
            int pend_blk = 0, pend_d = 0;
            // rows whose stores are committed but not yet published
            int pub_blk[kPublishBatch], pub_d[kPublishBatch], npub = 0;
            auto publish = [&]() {
                if (npub == 0) return;
                tma_store_wait<0>();          // the rows' bulk stores have been performed
                fence_proxy_async_all();
                fence_acq_rel_sys();          // ... and are ordered, with the table stores, before the counts
#pragma unroll
                for (int i = 0; i < kPublishBatch; ++i)
                    if (i < npub) red_add_relaxed_sys(reinterpret_cast<int*>(f.ctrl_ptrs[pub_d[i]] + f.off_blk_cnt) + pub_blk[i], 1);
                npub = 0;
            };
            auto store_pending = [&]() -> bool {
                if (!pend) return true;
                const uint32_t b = pend_b;
                if (!mbar_wait(dispatch_bar(warp, b), b ? ph1 : ph0, abort_flag, g.status, 640)) return false;
                if (b) ph1 ^= 1u; else ph0 ^= 1u;
                bulk_store_1d(pend_dst, buf0 + b * kDispatchChunk, pend_bytes);
                tma_store_commit();
                pend = false;
                if (pend_last) {
#pragma unroll
                    for (int i = 0; i < kPublishBatch; ++i)
                        if (i == npub) { pub_blk[i] = pend_blk; pub_d[i] = pend_d; }
                    if (++npub == kPublishBatch) publish();
                }
                return true;
            };
            for (int pos = wid; ok && pos < num_send; pos += warps_total) {
                const int entry = f.send_order[pos];
                const int t = entry / f.K, k = entry - t * f.K;
                const int e = (int)load_idx(f.topk_idx, f.idx_is64, entry);
                const int d = e / e_local;
                const int slot = f.send_slot[entry];
                if (slot < 0 || slot >= f.slot_cap || e < 0 || e >= f.E) continue;   // never store outside the destination table
                const uint64_t arena = f.arena_ptrs[d];
                const uint8_t* src = reinterpret_cast<const uint8_t*>(f.x) + (size_t)t * row_bytes;
                const uint64_t dst = arena + f.off_slot_x + (uint64_t)slot * row_bytes;
                for (uint32_t off = 0; off < row_bytes; off += kDispatchChunk) {
                    const uint32_t chunk = min((uint32_t)kDispatchChunk, row_bytes - off);
                    const uint32_t b = nchunk & 1u;
                    tma_store_wait_read<0>();            // the store that last used this buffer (the newest group) has read it out
                    mbar_arrive_expect_tx(dispatch_bar(warp, b), chunk);
                    bulk_load_1d(buf0 + b * kDispatchChunk, src + off, chunk, dispatch_bar(warp, b));
                    ++nchunk;
                    // the previous chunk sits in the other buffer
                    if (!(ok = store_pending())) break;
                    pend = true;
                    pend_b = b;
                    pend_dst = dst + off;
                    pend_bytes = chunk;
                    pend_last = off + kDispatchChunk >= row_bytes;
                    pend_blk = slot >> 7;
                    pend_d = d;
                    if (off == 0 && f.with_meta) {
                        const int row = f.send_row[(long)t * f.N + d];
                        reinterpret_cast<float*>(arena + f.off_slot_w)[slot] = f.topk_w[entry];
                        reinterpret_cast<int*>(arena + f.off_slot_tk)[slot] = entry;
                        reinterpret_cast<int*>(arena + f.off_slot_row)[slot] = row;
                        bool first = true;                       // first entry of token t that goes to rank d
                        for (int k2 = 0; k2 < k; ++k2) {
                            const long long e2 = load_idx(f.topk_idx, f.idx_is64, (long)t * f.K + k2);
                            if (e2 >= 0 && e2 < f.E && (int)e2 / e_local == d) first = false;
                        }
                        if (first) reinterpret_cast<int*>(arena + f.off_row_first)[row] = slot;
                    }
                }
            }
            if (ok) ok = store_pending();
            if (ok) publish();
            tma_store_wait<0>();              // nothing of this thread's copies is in flight past this point
        }
        __syncwarp();
        cluster_sync_all();                   // both CTAs of the pair are done with the staging buffers: they become operand stages
    }

    // ---------------------------------------------------------------------- compute role
    // Tiles are claimed in arrival order from one counter per launch (atomicAdd by the first CTA's producer thread,
    // one tile ahead) and handed to the other roles of the pair through a small ring in each CTA's shared memory,
    // so dispatch pairs simply join once their rows are out and uneven tiles balance themselves.
    {
        int num_units = g.max_units;
        if (g.num_units_dev != nullptr) num_units = min(*g.num_units_dev, g.max_units);
        const int nk = g.k_total / BK;
        const int total_tiles = num_units * g.num_n_blocks;
        const uint32_t ring_addr = bar_base + kRingOffset;
        volatile int* ring = reinterpret_cast<volatile int*>(smem_gen + kStagesF * kStageBytesF + kRingOffset);
        // consumer side of the ring: wait for entry `ss`, copy it, release the entry (to the first CTA's scheduler)
        auto next_tile = [&](int& ss, uint32_t& sph, int site, int& t) -> bool {
            if (!mbar_wait_cluster_acquire(sched_full(ss), sph, abort_flag, g.status, site)) return false;
            t = ring[ss];
            __syncwarp();
            if (lane == 0) {
                if (rank == 0) mbar_arrive(sched_empty(ss));
                else mbar_arrive_cluster(mapa_shared(sched_empty(ss), 0));
            }
            if (++ss == kSchedDepth) { ss = 0; sph ^= 1u; }
            return true;
        };

        if (warp == 0) {
            // -------------------------------------------------------------- tile scheduler (first CTA) + TMA producer
            if (elect_one()) {
                int stage = 0;
                uint32_t phase = 0;
                bool ok = true;
                TileF tile;
                int ss = 0;
                uint32_t sph = 0;
                int t_next = (rank == 0) ? atomicAdd(f.tile_counter, 1) : 0;
                while (ok) {
                    int t;
                    if (rank == 0) {
                        t = (t_next < total_tiles) ? t_next : -1;
                        if (t >= 0) t_next = atomicAdd(f.tile_counter, 1);   // its latency hides under this tile's loads
                        if (!mbar_wait(sched_empty(ss), sph ^ 1u, abort_flag, g.status, 650)) { ok = false; break; }
                        ring[ss] = t;
                        st_shared_cluster_u32(mapa_shared(ring_addr + 4u * ss, 1), (uint32_t)t);
                        mbar_arrive(sched_full(ss));
                        mbar_arrive_cluster_release(mapa_shared(sched_full(ss), 1));
                    } else {
                        if (!mbar_wait_cluster_acquire(sched_full(ss), sph, abort_flag, g.status, 651)) { ok = false; break; }
                        t = ring[ss];
                        mbar_arrive_cluster(mapa_shared(sched_empty(ss), 0));
                    }
                    if (++ss == kSchedDepth) { ss = 0; sph ^= 1u; }
                    if (t < 0) break;
                    get_tile_f(g, f.unit_order, t, total_tiles, num_units, tile);
                    const bool live = (rank == 0) || tile.two;
                    const int my_blk = tile.blk0 + (int)rank;
                    if (live) {
                        // rows of this block come from the peers' dispatch pairs: wait for all of them
                        const int le = g.mblock_expert[my_blk];
                        const int valid_end = f.seg_offsets[le] + f.expert_total_local[le];
                        const int need = max(0, min(128, valid_end - my_blk * 128));
                        if (!wait_flag_ge_sys(f.blk_cnt + my_blk, need, g.status, 600)) { *abort_flag = 1u; ok = false; break; }
                        fence_proxy_async_all();   // generic-proxy peer stores -> async-proxy (TMA) reads
                    }
                    const int m0 = my_blk * BM;
                    const int n0 = tile.n_blk * BN + (int)rank * (BN / 2);
                    for (int kb = 0; kb < nk; ++kb) {
                        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, g.status, 610)) { ok = false; break; }
                        const uint32_t a_dst = smem_base + stage * kStageBytesF;
                        const uint32_t b_dst = a_dst + kAStageBytes;
                        const uint32_t bar = mapa_shared(full_bar(stage), 0);
                        if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * kStageBytesF);
                        else mbar_arrive_cluster(bar);
                        const int k = kb * BK;
                        tma_load_2d_2cta(a_dst, &map_a, bar, k, m0);
                        if constexpr (!B_MN) {
                            tma_load_2d_2cta(b_dst, &map_b, bar, k, tile.group * g.b_group_rows + n0);
                        } else {
                            const int krow = tile.group * g.b_group_rows + k;
#pragma unroll
                            for (int a = 0; a < BN / 128; ++a) tma_load_2d_2cta(b_dst + a * kAtomBytes, &map_b, bar, n0 + 64 * a, krow);
                        }
                        if (++stage == kStagesF) { stage = 0; phase ^= 1u; }
                    }
                }
            }
        } else if (warp == 1 && rank == 0) {
            // -------------------------------------------------------------- UMMA issuer
            constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, false, B_MN);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int ss = 0;
            uint32_t sph = 0;
            for (int iter = 0; ok; ++iter) {
                int t;
                if (!next_tile(ss, sph, 652, t) || t < 0) break;
                const int as = iter & 1;
                const uint32_t aphase = (iter >> 1) & 1;
                if (!mbar_wait(tempty_bar(as), aphase ^ 1u, abort_flag, g.status, 620)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(as * BN);
                for (int kb = 0; kb < nk; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag, g.status, 621)) { ok = false; break; }
                    tcgen05_fence_after();
                    if (elect_one()) {
                        const uint32_t a_addr = smem_base + stage * kStageBytesF;
                        const uint32_t b_addr = a_addr + kAStageBytes;
#pragma unroll
                        for (int k = 0; k < BK / UK; ++k) {
                            const uint64_t a_desc = make_smem_desc_sw128(a_addr + k * (UK * 2), 0, 1024);
                            const uint64_t b_desc = B_MN ? make_smem_desc_sw128(b_addr + k * (UK * 128), kAtomBytes, 1024)
                                                         : make_smem_desc_sw128(b_addr + k * (UK * 2), 0, 1024);
                            umma_bf16_ss_2cta(d_tmem, a_desc, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                        }
                        umma_commit_2cta(empty_bar(stage), 3u);
                        if (kb == nk - 1) umma_commit_2cta(tfull_bar(as), 3u);
                    }
                    __syncwarp();
                    if (++stage == kStagesF) { stage = 0; phase ^= 1u; }
                }
            }
        } else if (warp >= 4) {
            // -------------------------------------------------------------- epilogue
            const int q = warp & 3;
            const int h = (warp - 4) >> 2;
            const int r = q * 32 + lane;
            bool ok = true;
            TileF tile;
            int ss = 0;
            uint32_t sph = 0;
            for (int iter = 0; ok; ++iter) {
                int t;
                if (!next_tile(ss, sph, 653, t) || t < 0) break;
                get_tile_f(g, f.unit_order, t, total_tiles, num_units, tile);
                const int as = iter & 1;
                const uint32_t aphase = (iter >> 1) & 1;
                if (!mbar_wait(tfull_bar(as), aphase, abort_flag, g.status, 630)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t taddr0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(as * BN + h * (BN / 2));
                const int n0 = tile.n_blk * BN + h * (BN / 2);
                const bool live = (rank == 0) || tile.two;
                const long row = (long)(tile.blk0 + (int)rank) * BM + r;
                if (live) epilogue_thread<EPI>(g, taddr0, row, true, n0, tile.n_blk * 2 + h, false);
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(mapa_shared(tempty_bar(as), 0));
            }
        }
    }

    tcgen05_fence_before();
    cluster_sync_all();
    if (warp == 2) {
        tcgen05_fence_after();
        tmem_dealloc_2cta(tmem_base, kTmemCols);
    }
}

template <bool B_MN, int EPI>
cudaError_t launch_fused(const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& g, const FusedArgs& f, int num_sms,
                         cudaStream_t stream) {
    auto kern = fused_dispatch_gemm_kernel<B_MN, EPI>;
    static bool configured[64] = {};
    if (cudaError_t e = ensure_smem_limit(kern, kSmemBytesF, configured); e != cudaSuccess) return e;
    int grid = num_sms & ~1;
    if (grid < 2 * (f.num_dispatch_clusters + 1)) return cudaErrorInvalidConfiguration;
    // All CTAs must be resident at once (compute pairs wait for rows that dispatch pairs of OTHER ranks send,
    // and this rank's dispatch pairs serve the others): a cooperative launch makes the runtime check that.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytesF;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;
    at[0].val.cooperative = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, ma, mb, g, f);
}

}  // namespace

cudaError_t fused_dispatch_gemm(int kind, const void* slot_x, int slot_rows, const void* w, const GemmArgsPublic& p, const FusedArgs& f,
                                int num_sms, cudaStream_t stream) {
    // kind 0: forward gate_up + SwiGLU (W_gateup [E*2I, H] K-major);  kind 1: backward grad_act + dSwiGLU (W_down [E*H, I] MN-major)
    if (p.H % BK != 0 || p.I % 32 != 0 || slot_rows % BM != 0 || slot_rows <= 0) return cudaErrorInvalidValue;
    if (reinterpret_cast<uintptr_t>(f.x) % 16 != 0 || f.off_slot_x % 16 != 0) return cudaErrorInvalidValue;   // bulk copies need 16-byte alignment
    CUtensorMap ma, mb;
    cudaError_t e;
    if ((e = make_map(&ma, slot_x, (uint64_t)slot_rows, p.H, BK, BM)) != cudaSuccess) return e;
    GemmArgs g{};
    g.k_total = p.H;
    g.max_mblocks = slot_rows / BM;
    g.num_mblocks_dev = p.lay.num_mblocks_dev;
    g.mblock_expert = p.lay.mblock_expert;
    g.unit_blk = p.lay.unit_blk;
    g.num_units_dev = p.lay.num_units_dev;
    g.max_units = p.lay.max_units;
    g.row_w = p.row_w;
    g.status = p.status;
    const int sms = default_sms(num_sms);
    if (kind == 0) {
        if ((e = make_map(&mb, w, (uint64_t)p.num_local_experts * 2 * p.I, p.H, BK, BN / 2)) != cudaSuccess) return e;
        g.n_total = 2 * p.I;
        g.num_n_blocks = (2 * p.I + BN - 1) / BN;
        g.b_group_rows = 2 * p.I;
        g.d = static_cast<__nv_bfloat16*>(p.out0);      // act
        g.ldd = p.I;
        g.aux = static_cast<__nv_bfloat16*>(p.out1);    // preact
        g.ld_aux = 2 * p.I;
        return launch_fused<false, kEpiSwiGLU>(ma, mb, g, f, sms, stream);
    }
    if ((e = make_map(&mb, w, (uint64_t)p.num_local_experts * p.H, p.I, 64, BK)) != cudaSuccess) return e;
    g.n_total = p.I;
    g.num_n_blocks = (p.I + BN - 1) / BN;
    g.b_group_rows = p.H;
    g.d = static_cast<__nv_bfloat16*>(p.out0);          // act_w
    g.ldd = p.I;
    g.aux = static_cast<__nv_bfloat16*>(p.out1);        // dGU
    g.ld_aux = 2 * p.I;
    g.preact = static_cast<const __nv_bfloat16*>(p.preact);
    g.droute_part = p.droute_part;
    g.n_parts = 2 * ((p.I + BN - 1) / BN);
    return launch_fused<true, kEpiDSwiGLU>(ma, mb, g, f, sms, stream);
}

}  // namespace tmoe
