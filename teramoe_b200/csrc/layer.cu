// Whole-layer kernel: ONE cooperative persistent launch per direction.
//
// Every CTA pair (thread-block cluster of two, tcgen05 cta_group::2) is a worker that takes items from a work
// list in order (one atomic counter per launch).  The list is built on the device by the scheduler kernel below
// and decides the schedule; the roles are
//
//   dispatch   the first `num_dispatch_clusters` pairs first stream this rank's routed rows straight into their
//              final slot of the destination ranks' operand table (bulk copies through shared memory) and bump
//              the destination's per-128-row arrival counters; then they become workers like the others.
//              With `wire_rank` a token's row crosses the link once per destination rank: it goes to the entry
//              with the smallest slot there, the token's other entries on that rank only get their table entries,
//              and the receiver's gather warps copy the row into those slots (`replicate`) before the block counts
//              as ready (reference: one message per (token, rank) and a local replicate,
//              csrc/kernels/layout.cu:79-95, csrc/teramoe/teramoe_orchestrator.cu:1216-1269).
//   scheduler  `layer_schedule_kernel`: orders the items.  Units (one or two 128-row blocks of one expert) are
//              taken in arrival order and cut into batches of `group_units`; a batch's second GEMM follows its
//              first GEMM at a distance of `lag_percent` of the next batch, so the intermediate activation is
//              still in L2 and the pushed rows are spread over the whole kernel instead of one burst.
//   compute    first GEMM (forward: gate_up + SwiGLU x route, pre-activation side store; backward: grad_act with
//              the dSwiGLU epilogue) waits for the arrival counters of its rows; second GEMM (down / dX) waits for
//              the per-unit completion counter of the first GEMM and reads the activation back from L2.
//   combine    the second GEMM's epilogue: every output row leaves for the token's rank as bulk copies shared ->
//              peer global (plus, in backward, the row's route-weight gradient).  When a rank's last pushed tile is
//              complete it tells every rank (release store at system scope).
//   wgrad      backward: the two weight-gradient GEMMs (varlen-K, both operands MN-major) as the tail of the list.
//   gather     warps 2 and 3 of every CTA (joined by the epilogue warps when the list is exhausted): once every rank has
//              said that its pushes are complete, sum each token's landed rows in fp32 and write the output row
//              (backward: also the route-weight gradients).  In backward this runs under the weight-gradient GEMMs.
//
// Reference counterpart: teramoe_fused_forward_kernel / teramoe_fused_backward_kernel with their dispatch, scheduler,
// compute, combine and gather SM roles (csrc/teramoe/teramoe_orchestrator.cu:2978-3042, :4880-4936, :524-1369,
// :1482-1624, :1626-1907, :1923-2812, :2849-2976, :4495-4848).  Differences: rows go to their final slot (no rings,
// no publisher warps), SMs are not partitioned by role (every pair takes whatever item is next, so nothing idles),
// the schedule is data written by a scheduler kernel instead of a scheduler SM polling queues, the weight gradients
// run inside the launch, and every wait is bounded.
#include "layer.h"

#include "gemm_common.cuh"

namespace tmoe {

using namespace detail;

namespace {

constexpr int kStagesL = 5;
constexpr int kBHalfBytesL = (BN / 2) * BK * 2;
constexpr int kStageBytesL = kAStageBytes + kBHalfBytesL;                 // 32 KB
constexpr int kPipeBytesL = kStagesL * kStageBytesL;                      // 160 KB
constexpr int kPushBytesL = kEpiWarps * kPushWarpBytes;                   // 36 KB
constexpr int kBarOffsetL = kPipeBytesL + kPushBytesL;
constexpr int kSmemBytesL = kBarOffsetL + 512 + 1024;
constexpr int kDispatchChunkL = 8192;                                     // two per dispatch warp
constexpr int kPublishBatchL = 4;
constexpr int kSchedDepthL = 4;
constexpr int kGatherChunk = 4;                                           // tokens a gather warp claims at a time
constexpr uint32_t kOffTmemSlot = 112, kOffDispatchBar = 128, kOffSchedFull = 320, kOffSchedEmpty = 352, kOffRing = 384;
constexpr uint32_t kSchedConsumersL = 2 * kEpiWarps + 2;
static_assert((kThreads / 32) * 2 * kDispatchChunkL <= kBarOffsetL, "dispatch staging exceeds the operand stages + push staging");
static_assert(8 * (2 * kStagesL + 4) <= (int)kOffTmemSlot, "pipeline barriers overlap the flags");

// One grouped GEMM of the work list.
struct LayerPhase {
    alignas(64) CUtensorMap map_a;
    alignas(64) CUtensorMap map_b;
    GemmArgs g;
};

struct LayerArgs {
    LayerPhase ph[4];
    FusedArgs f;
    __nv_bfloat16* slot_x;       // this rank's operand table (the replicate role copies rows inside it)
    const int4* work;
    const int* num_work;
    int max_work;
    const int2* expert_units;
    int* item_counter;
    int* push_done;
    int* units_complete;         // units whose first GEMM is complete
    int* gather_counter;         // next token of the gather role
    // backward: the gather warps first rebuild X in slot space (operand of dW_gateup) from the rows kept by forward
    const __nv_bfloat16* x_rows; // [rows, H] one row per received token
    const int* x_slot_row;       // [slots] row of x_rows that feeds each slot (-1: zero row)
    __nv_bfloat16* xperm;        // [slots, H]
    int expand_rows;             // slots to fill
    int* expand_counter;         // next slot to claim
    int* expand_done;            // slots filled
    int* unit_done;
    const uint64_t* signal_ptrs;
    const int* my_signal;
    int rank, N, epoch;
    const __nv_bfloat16* landing;
    __nv_bfloat16* out;
    const float* gtw_in;
    float* gtw_out;
    unsigned long long* stats;   // optional [kLayerStatWords] time counters (ns summed over the waiting threads), see layer.h
    const int* geom_ok;          // optional: 0 = the tables were sized too small for this call's layout (every rank sees the same)
    int* status;
};

__device__ __forceinline__ long long load_idx_l(const void* idx, int is64, long i) {
    return is64 ? reinterpret_cast<const long long*>(idx)[i] : (long long) reinterpret_cast<const int*>(idx)[i];
}
__device__ __forceinline__ void red_add_relaxed_sys_l(int* p, int v) {
    asm volatile("red.relaxed.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int atom_add_acq_rel_gpu(int* p, int v) {
    int old;
    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ int4 ld_cg_v4(const void* p) {
    int4 v;
    // volatile keeps it behind the acquire loads that precede it; no memory clobber, so that many can be in flight
    asm volatile("ld.global.cg.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void accum8(float (&acc)[8], const int4& v) {
    const uint32_t u[4] = {(uint32_t)v.x, (uint32_t)v.y, (uint32_t)v.z, (uint32_t)v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = unpack_bf16x2(u[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
    }
}
__device__ __forceinline__ int4 pack8(const float (&acc)[8]) {
    return make_int4((int)pack_bf16x2(acc[0], acc[1]), (int)pack_bf16x2(acc[2], acc[3]), (int)pack_bf16x2(acc[4], acc[5]),
                     (int)pack_bf16x2(acc[6], acc[7]));
}

// Bounded wait until *flag >= target (acquire, GPU scope): counters that other SMs of this GPU bump.  The limit is
// the one for waits on other ranks, because what is awaited depends on rows that other ranks send.
__device__ __forceinline__ bool wait_flag_ge_gpu(const int* flag, int target, int* status, int site) {
    if (ld_acquire_gpu(flag) >= target) return true;
    const uint64_t limit_ns = peer_wait_limit_ns(status);
    const uint64_t t0 = globaltimer_ns();
#pragma unroll 1
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i) {
            if (ld_acquire_gpu(flag) >= target) return true;
            __nanosleep(64);
        }
        if (status != nullptr && ld_relaxed_sys(status) != 0) return false;
        if (globaltimer_ns() - t0 > limit_ns) {
            report_status(status, kStatusFlagTimeout, site, target);
            return false;
        }
    }
}

// Work items carry their whole geometry (the scheduler kernel looks the tables up once), so no role of a pair
// has to load anything from global memory between taking an item and working on it:
//   x  bits 0-3 kind, bit 4 "the unit has two blocks", bits 8-27 local expert
//   first / second GEMM:  y = unit, z = column block | rows awaited in block 0 << 16 | rows awaited in block 1 << 24, w = first block
//   weight gradients:     y = first slot row of the expert, z = column block | row unit of dW << 16, w = number of 64-row K blocks
struct ItemGeom {
    int kind, n_blk, group, k0, nk, m0, unit, need;
    bool live;      // this CTA's 128 rows are real
    long row0;      // first output row of this CTA (M-grouped) or of dW (weight gradient)
    int m_in_group; // weight gradient: first dW row of this CTA inside the expert
};

__device__ __forceinline__ int item_kind(const int4& it) { return it.x < 0 ? -1 : (it.x & 15); }

__device__ __forceinline__ void item_geometry(const LayerArgs& L, const int4& it, uint32_t rank, ItemGeom& q) {
    q.kind = it.x & 15;
    q.group = (it.x >> 8) & 0xfffff;
    const GemmArgs& g = L.ph[q.kind].g;
    if (q.kind <= kWorkGemm2) {
        q.unit = it.y;
        q.n_blk = it.z & 0xffff;
        q.need = rank == 0 ? ((it.z >> 16) & 0xff) : ((it.z >> 24) & 0xff);
        q.live = (rank == 0) || ((it.x >> 4) & 1);
        q.m0 = (it.w + (int)rank) * BM;
        q.row0 = (long)q.m0;
        q.k0 = 0;
        q.nk = g.k_total / BK;
        q.m_in_group = 0;
    } else {
        q.unit = -1;
        q.need = 0;
        q.n_blk = it.z & 0xffff;
        q.live = true;
        q.m_in_group = ((it.z >> 16) * 2 + (int)rank) * BM;
        q.m0 = q.m_in_group;
        q.row0 = (long)q.group * g.m_total + q.m_in_group;
        q.k0 = it.y;
        q.nk = it.w;
    }
}

template <bool BWD>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
moe_layer_kernel(const __grid_constant__ LayerArgs L) {
    if (L.geom_ok != nullptr && *L.geom_ok == 0) return;      // before anything is allocated or sent; the host repeats the call
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t push_stage_base = smem_base + kPipeBytesL;
    const uint32_t bar_base = smem_base + kBarOffsetL;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStagesL + s); };
    auto tfull_bar = [&](int s) { return bar_base + 8u * (2 * kStagesL + s); };
    auto tempty_bar = [&](int s) { return bar_base + 8u * (2 * kStagesL + 2 + s); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + kBarOffsetL + kOffTmemSlot);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    auto dispatch_bar = [&](int w, uint32_t b) { return bar_base + kOffDispatchBar + 8u * (2u * w + b); };
    auto sched_full = [&](int e) { return bar_base + kOffSchedFull + 8u * e; };
    auto sched_empty = [&](int e) { return bar_base + kOffSchedEmpty + 8u * e; };

    const FusedArgs& f = L.f;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int cluster_id = blockIdx.x >> 1;
    const int cd = f.num_dispatch_clusters;
    const bool is_dispatch = cluster_id < cd;

    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        for (int s = 0; s < kStagesL; ++s) {
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
        for (int e = 0; e < kSchedDepthL; ++e) {
            mbar_init(sched_full(e), 1);
            mbar_init(sched_empty(e), kSchedConsumersL);
        }
        fence_mbar_init();
#pragma unroll
        for (int p = 0; p < (BWD ? 4 : 2); ++p) {
            tma_prefetch_desc(&L.ph[p].map_a);
            tma_prefetch_desc(&L.ph[p].map_b);
        }
    }
    if (warp == 2) tmem_alloc_2cta(smem_u32((const void*)tmem_slot), kTmemCols);
    tcgen05_fence_before();
    cluster_sync_all();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    int num_units = L.ph[0].g.max_units;
    if (L.ph[0].g.num_units_dev != nullptr) num_units = min(*L.ph[0].g.num_units_dev, num_units);
    const int nb1 = L.ph[0].g.num_n_blocks;                       // column blocks of the first GEMM
    const int unit_target = 2 * kEpiWarps * nb1;                  // epilogue warps that finish a unit's first GEMM
    const int push_target = 2 * kEpiWarps * num_units * L.ph[1].g.num_n_blocks;
    auto signal_ranks = [&]() {
        // this rank's pushed rows are complete and (by the fences of the warps that counted) visible: tell every rank
        fence_acq_rel_sys();
        for (int d = 0; d < L.N; ++d) st_release_sys(reinterpret_cast<int*>(L.signal_ptrs[d]) + L.rank, L.epoch);
    };
    if (blockIdx.x == 0 && threadIdx.x == 0 && push_target == 0) signal_ranks();   // nothing to push: say so at once

    if (is_dispatch) {
        // ------------------------------------------------------------------ dispatch role (all 12 warps)
        // Each warp owns two 8 KB staging buffers in the (not yet used) operand stages.  Its leader streams the
        // rows through them in chunks with bulk copies: global -> shared (completes on the buffer's mbarrier),
        // shared -> the destination's slot row (bulk group); the load of chunk c runs while chunk c-1 is stored.
        // Rows are published in batches (arrival counter of the row's 128-row block at the destination):
        // bulk-group wait, one system-scope fence, one red.add per row.
        const int num_send = min(*f.num_send, f.max_send);
        const int warps_total = cd * 2 * (kThreads / 32);
        const int wid = (cluster_id * 2 + (int)rank) * (kThreads / 32) + warp;
        const int e_local = f.E / f.N;
        if (lane == 0) {
            const uint32_t buf0 = smem_base + (uint32_t)warp * (2 * kDispatchChunkL);
            const uint32_t row_bytes = (uint32_t)f.H * 2u;
            uint32_t ph0 = 0, ph1 = 0, nchunk = 0;
            bool ok = true;
            bool pend = false, pend_last = false;
            uint64_t pend_dst = 0;
            uint32_t pend_bytes = 0, pend_b = 0;
            int pend_blk = 0, pend_d = 0, pend_entry = 0;
            int pub_blk[kPublishBatchL], pub_d[kPublishBatchL], npub = 0;
            auto publish = [&]() {
                if (npub == 0) return;
                tma_store_wait<0>();
                fence_proxy_async_all();
                fence_acq_rel_sys();
#pragma unroll
                for (int i = 0; i < kPublishBatchL; ++i)
                    if (i < npub) red_add_relaxed_sys_l(reinterpret_cast<int*>(f.ctrl_ptrs[pub_d[i]] + f.off_blk_cnt) + pub_blk[i], 1);
                npub = 0;
            };
            auto add_publish = [&](int blk, int d) {
#pragma unroll
                for (int i = 0; i < kPublishBatchL; ++i)
                    if (i == npub) { pub_blk[i] = blk; pub_d[i] = d; }
                if (++npub == kPublishBatchL) publish();
            };
            // wire_rank: slot of entry (t, k2) if it is another entry of token t on rank d (a sibling of the home entry), else -1
            auto sibling_slot = [&](int t, int k, int k2, int d) -> int {
                if (k2 == k) return -1;
                const long long e2 = load_idx_l(f.topk_idx, f.idx_is64, (long)t * f.K + k2);
                if (e2 < 0 || e2 >= f.E || (int)e2 / e_local != d) return -1;
                const int s2 = f.send_slot[(long)t * f.K + k2];
                return (s2 >= 0 && s2 < f.slot_cap) ? s2 : -1;
            };
            auto store_pending = [&]() -> bool {
                if (!pend) return true;
                const uint32_t b = pend_b;
                if (!mbar_wait(dispatch_bar(warp, b), b ? ph1 : ph0, abort_flag, L.status, 640)) return false;
                if (b) ph1 ^= 1u; else ph0 ^= 1u;
                bulk_store_1d(pend_dst, buf0 + b * kDispatchChunkL, pend_bytes);
                tma_store_commit();
                pend = false;
                if (pend_last) {
                    add_publish(pend_blk, pend_d);
                    if (f.wire_rank) {
                        // the row also stands for the token's other entries on that rank: their blocks count it too, and the
                        // counts go out behind the same completed copy and fence as the home's
                        const int t = pend_entry / f.K, k = pend_entry - t * f.K;
                        for (int k2 = 0; k2 < f.K; ++k2) {
                            const int s2 = sibling_slot(t, k, k2, pend_d);
                            if (s2 >= 0) add_publish(s2 >> 7, pend_d);
                        }
                    }
                }
                return true;
            };
            for (int pos = wid; ok && pos < num_send; pos += warps_total) {
                const int entry = f.send_order[pos];
                const int t = entry / f.K, k = entry - t * f.K;
                const int e = (int)load_idx_l(f.topk_idx, f.idx_is64, entry);
                const int slot = f.send_slot[entry];
                if (slot < 0 || slot >= f.slot_cap || e < 0 || e >= f.E) continue;   // never store outside the destination table
                const int d = e / e_local;
                if (f.wire_rank) {
                    // only the home entry of (t, d) travels: the one with the smallest slot, which is also the first of them
                    // in sending order and the first the receiver works on
                    bool home = true;
                    for (int k2 = 0; k2 < f.K; ++k2) {
                        const int s2 = sibling_slot(t, k, k2, d);
                        if (s2 >= 0 && s2 < slot) home = false;
                    }
                    if (!home) continue;
                }
                const uint64_t arena = f.arena_ptrs[d];
                const uint8_t* src = reinterpret_cast<const uint8_t*>(f.x) + (size_t)t * row_bytes;
                const uint64_t dst = arena + f.off_slot_x + (uint64_t)slot * row_bytes;
                for (uint32_t off = 0; off < row_bytes; off += kDispatchChunkL) {
                    const uint32_t chunk = min((uint32_t)kDispatchChunkL, row_bytes - off);
                    const uint32_t b = nchunk & 1u;
                    tma_store_wait_read<0>();
                    mbar_arrive_expect_tx(dispatch_bar(warp, b), chunk);
                    bulk_load_1d(buf0 + b * kDispatchChunkL, src + off, chunk, dispatch_bar(warp, b));
                    ++nchunk;
                    if (!(ok = store_pending())) break;
                    pend = true;
                    pend_b = b;
                    pend_dst = dst + off;
                    pend_bytes = chunk;
                    pend_last = off + kDispatchChunkL >= row_bytes;
                    pend_blk = slot >> 7;
                    pend_d = d;
                    pend_entry = entry;
                    if (off == 0 && f.wire_rank) {
                        // where every slot of (t, d) gets its row from, and the table entries of the slots that get no row
                        const int row = f.send_row[(long)t * f.N + d];
                        reinterpret_cast<int*>(arena + f.off_slot_src)[slot] = -1;
                        for (int k2 = 0; k2 < f.K; ++k2) {
                            const int s2 = sibling_slot(t, k, k2, d);
                            if (s2 < 0) continue;
                            reinterpret_cast<int*>(arena + f.off_slot_src)[s2] = slot;
                            if (f.with_meta) {
                                reinterpret_cast<float*>(arena + f.off_slot_w)[s2] = f.topk_w[(long)t * f.K + k2];
                                reinterpret_cast<int*>(arena + f.off_slot_tk)[s2] = t * f.K + k2;
                                reinterpret_cast<int*>(arena + f.off_slot_row)[s2] = row;
                            }
                        }
                    }
                    if (off == 0 && f.with_meta) {
                        const int row = f.send_row[(long)t * f.N + d];
                        reinterpret_cast<float*>(arena + f.off_slot_w)[slot] = f.topk_w[entry];
                        reinterpret_cast<int*>(arena + f.off_slot_tk)[slot] = entry;
                        reinterpret_cast<int*>(arena + f.off_slot_row)[slot] = row;
                        bool first = true;                       // first entry of token t that goes to rank d (wire_rank: the home is the only one)
                        for (int k2 = 0; k2 < k && !f.wire_rank; ++k2) {
                            const long long e2 = load_idx_l(f.topk_idx, f.idx_is64, (long)t * f.K + k2);
                            if (e2 >= 0 && e2 < f.E && (int)e2 / e_local == d) first = false;
                        }
                        if (first) reinterpret_cast<int*>(arena + f.off_row_first)[row] = slot;
                    }
                }
            }
            if (ok) ok = store_pending();
            if (ok) publish();
            tma_store_wait<0>();
        }
        __syncwarp();
        cluster_sync_all();                   // both CTAs of the pair are done with the staging buffers: they become operand stages
    }

    // ---------------------------------------------------------------------- gather role
    // Sums each token's landed rows once every rank has said that its pushes are complete.  Warps 2 and 3 of every CTA
    // do nothing else (in backward their memory traffic runs under the weight-gradient GEMMs); the epilogue warps join
    // when the work list is exhausted.  Token chunks come from their own counter.
    auto replicate_loop = [&]() {
        // wire_rank: units in arrival order; when the rows of a block have been counted in (rows that arrived, and for the
        // others the word that says which slot holds their row, sent behind that row), copy the missing rows and
        // declare the block ready.  The first GEMM's producers wait for `blk_ready` instead of the arrival counters.
        const int nvec = f.H / 8;
        const GemmArgs& g0 = L.ph[0].g;
        const int* slot_src = f.slot_src;
        while (true) {
            int i = 0;
            if (lane == 0) i = atomicAdd(f.replicate_counter, 1);
            i = __shfl_sync(0xffffffffu, i, 0);
            if (i >= num_units) break;
            const int u = f.unit_order[i];
            const int b0 = g0.unit_blk[u], b1 = g0.unit_blk[u + 1];
            for (int b = b0; b < b1; ++b) {
                const int le = g0.mblock_expert[b];
                const int valid_end = f.seg_offsets[le] + f.expert_total_local[le];
                const int need = max(0, min(128, valid_end - b * 128));
                if (need == 0) continue;
                int got = 1;
                if (lane == 0) got = wait_flag_ge_sys(f.blk_cnt + b, need, L.status, 604) ? 1 : 0;
                got = __shfl_sync(0xffffffffu, got, 0);
                __syncwarp();                                       // the other lanes read behind lane 0's acquire
                if (!got) return;                                   // reported; the producers' wait on blk_ready runs out the same way
                for (int r = 0; r < need; ++r) {
                    const int sl = b * 128 + r;
                    const int src = __ldcg(slot_src + sl);
                    if (src < 0 || src >= f.slot_cap || src == sl) continue;
                    const int4* srow = reinterpret_cast<const int4*>(L.slot_x + (long)src * f.H);
                    int4* drow = reinterpret_cast<int4*>(L.slot_x + (long)sl * f.H);
                    for (int v = lane; v < nvec; v += 128) {          // four 16-byte loads in flight per lane
                        int4 t0 = ld_cg_v4(srow + v), t1 = make_int4(0, 0, 0, 0), t2 = t1, t3 = t1;
                        if (v + 32 < nvec) t1 = ld_cg_v4(srow + v + 32);
                        if (v + 64 < nvec) t2 = ld_cg_v4(srow + v + 64);
                        if (v + 96 < nvec) t3 = ld_cg_v4(srow + v + 96);
                        drow[v] = t0;
                        if (v + 32 < nvec) drow[v + 32] = t1;
                        if (v + 64 < nvec) drow[v + 64] = t2;
                        if (v + 96 < nvec) drow[v + 96] = t3;
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    fence_acq_rel_gpu();
                    red_add_release_gpu(f.blk_ready + b, need);
                }
            }
        }
    };
    auto expand_loop = [&]() {
        // X back into slot space, eight rows per claim, four 16-byte loads in flight per lane
        const int nvec = f.H / 8;
        while (true) {
            int s0 = 0;
            if (lane == 0) s0 = atomicAdd(L.expand_counter, 8);
            s0 = __shfl_sync(0xffffffffu, s0, 0);
            if (s0 >= L.expand_rows) break;
            const int s1 = min(s0 + 8, L.expand_rows);
            for (int sl = s0; sl < s1; ++sl) {
                const int rr = L.x_slot_row[sl];
                int4* dst = reinterpret_cast<int4*>(L.xperm + (long)sl * f.H);
                if (rr >= 0) {
                    warp_copy_row(dst, reinterpret_cast<const int4*>(L.x_rows + (long)rr * f.H), nvec, lane);
                } else {
                    for (int i = lane; i < nvec; i += 32) dst[i] = make_int4(0, 0, 0, 0);
                }
            }
            __syncwarp();
            if (lane == 0) {
                fence_acq_rel_gpu();
                red_add_release_gpu(L.expand_done, s1 - s0);
            }
        }
    };
    auto gather_loop = [&]() {
        const int K = f.K, H = f.H, nvec = f.H / 8;
        if (f.T <= 0) return;
        {
            // wait (bounded, slow polling: it may take most of the kernel) for every rank's signal
            const uint64_t limit_ns = peer_wait_limit_ns(L.status);
            const uint64_t t0 = globaltimer_ns();
            while (true) {
                const bool mine = lane >= L.N || ld_acquire_sys(L.my_signal + lane) >= L.epoch;
                if (__all_sync(0xffffffffu, mine)) break;
                if (ld_relaxed_sys(L.status) != 0) return;                    // someone gave up: unwind
                if (globaltimer_ns() - t0 > limit_ns) {
                    if (!mine) report_status(L.status, kStatusFlagTimeout, 660 + lane, L.epoch);
                    return;
                }
                __nanosleep(2000);
            }
            if (L.stats != nullptr && lane == 0 && warp == 2 && rank == 0) atomicAdd(L.stats + kStatWaitLanded, globaltimer_ns() - t0);
        }
        const bool stamps = L.stats != nullptr && lane == 0;
        if (stamps) atomicMax(L.stats + kStatKindFirst + kWorkReduce, ~globaltimer_ns());
        while (true) {
            int t0 = 0;
            if (lane == 0) t0 = atomicAdd(L.gather_counter, kGatherChunk);
            t0 = __shfl_sync(0xffffffffu, t0, 0);
            if (t0 >= f.T) break;
            for (int t = t0; t < min(t0 + kGatherChunk, f.T); ++t) {
                long long e = -1;
                if (lane < K) e = load_idx_l(f.topk_idx, f.idx_is64, (long)t * K + lane);
                const bool v = e >= 0 && e < f.E;
                const uint32_t valid = __ballot_sync(0xffffffffu, v);
                if constexpr (BWD) {
                    if (lane < K) L.gtw_out[(long)t * K + lane] = v ? __ldcg(L.gtw_in + (long)t * K + lane) : 0.f;
                }
                int4* dst = reinterpret_cast<int4*>(L.out + (long)t * H);
                const int4* base = reinterpret_cast<const int4*>(L.landing + (long)t * K * H);
                // Few warps per SM take part, so every lane keeps up to 16 loads in flight: the rows of eight entries
                // at two positions are all requested before the first is used.  Sum order: k ascending.
                for (int i = lane; i < nvec; i += 64) {
                    const bool two = i + 32 < nvec;
                    float a0[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                    float a1[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                    for (int k0 = 0; k0 < K; k0 += 8) {
                        int4 v0[8], v1[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const bool on = (valid >> (k0 + j)) & 1u;
                            const int4* row = base + (long)(k0 + j) * nvec;
                            v0[j] = on ? ld_cg_v4(row + i) : make_int4(0, 0, 0, 0);
                            v1[j] = (on && two) ? ld_cg_v4(row + i + 32) : make_int4(0, 0, 0, 0);
                        }
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            if ((valid >> (k0 + j)) & 1u) {
                                accum8(a0, v0[j]);
                                accum8(a1, v1[j]);
                            }
                        }
                    }
                    dst[i] = pack8(a0);
                    if (two) dst[i + 32] = pack8(a1);
                }
            }
        }
        if (stamps) atomicMax(L.stats + kStatKindLast + kWorkReduce, globaltimer_ns());
    };

    // ---------------------------------------------------------------------- worker roles
    {
        const int total_items = min(*L.num_work, L.max_work);
        const uint32_t ring_addr = bar_base + kOffRing;
        volatile int* ring = reinterpret_cast<volatile int*>(smem_gen + kBarOffsetL + kOffRing);
        // consumer side of the item ring: wait for entry `ss`, copy it, release the entry (to the first CTA's scheduler)
        // (the first CTA's entries are written by its own producer thread, the second CTA's arrive through the async proxy
        // and are counted on the barrier: a plain wait sees them, no cluster-scope fence anywhere)
        auto next_item = [&](int& ss, uint32_t& sph, int site, int4& it) -> bool {
            if (!mbar_wait(sched_full(ss), sph, abort_flag, L.status, site)) return false;
            it = make_int4(ring[4 * ss], ring[4 * ss + 1], ring[4 * ss + 2], ring[4 * ss + 3]);
            __syncwarp();
            if (lane == 0) {
                if (rank == 0) mbar_arrive(sched_empty(ss));
                else mbar_arrive_cluster(mapa_shared(sched_empty(ss), 0));
            }
            if (++ss == kSchedDepthL) { ss = 0; sph ^= 1u; }
            return true;
        };

        if (warp == 0) {
            // -------------------------------------------------------------- item fetch (first CTA) + TMA producer
            if (elect_one()) {
                int stage = 0;
                uint32_t phase = 0;
                bool ok = true;
                int ss = 0;
                uint32_t sph = 0;
                // The first CTA's producer claims items (one atomic per item, issued one item ahead) and hands them to
                // every role of the pair through the ring.  Both producers look at the NEXT item while the loads of the
                // current one are in flight: they fetch it and test what its operands wait for, so that between two
                // items the producer normally has nothing to wait for.
                int t_claim = (rank == 0) ? atomicAdd(L.item_counter, 1) : 0;
                unsigned long long w_arrive = 0, w_unit = 0, w_wgrad = 0;
                bool wgrad_ready = false;                    // every unit's first GEMM is complete (checked once per pair)
                bool wgrad_fenced = false;
                bool xperm_ready = false;
                int4 cur = make_int4(-1, 0, 0, 0), nxt = cur;
                bool have = false, nxt_ready = false;
                // 1: got an item, 0: none yet (non-blocking form, second CTA), -1: a wait ran out
                auto get_item = [&](int4& it, bool blocking) -> int {
                    if (rank == 0) {
                        it = (t_claim < total_items) ? L.work[t_claim] : make_int4(-1, 0, 0, 0);
                        if (it.x >= 0) t_claim = atomicAdd(L.item_counter, 1);      // needed when the next item is fetched
                        if (!mbar_wait(sched_empty(ss), sph ^ 1u, abort_flag, L.status, 650)) return -1;
                        ring[4 * ss] = it.x; ring[4 * ss + 1] = it.y; ring[4 * ss + 2] = it.z; ring[4 * ss + 3] = it.w;
                        mbar_arrive(sched_full(ss));
                        const uint32_t remote_bar = mapa_shared(sched_full(ss), 1);
                        mbar_arrive_expect_tx_cluster(remote_bar, 16u);
                        st_async_v4_cluster(mapa_shared(ring_addr + 16u * ss, 1), it, remote_bar);
                    } else {
                        if (blocking) {
                            if (!mbar_wait(sched_full(ss), sph, abort_flag, L.status, 651)) return -1;
                        } else if (!mbar_try_wait(sched_full(ss), sph)) {
                            return 0;
                        }
                        it = make_int4(ring[4 * ss], ring[4 * ss + 1], ring[4 * ss + 2], ring[4 * ss + 3]);
                        mbar_arrive_cluster(mapa_shared(sched_empty(ss), 0));
                    }
                    if (++ss == kSchedDepthL) { ss = 0; sph ^= 1u; }
                    return 1;
                };
                // what the operands of an item wait for; `block`: wait (bounded) instead of only looking
                auto operands_ready = [&](const ItemGeom& q, bool block) -> int {
                    if (q.kind == kWorkGemm1) {
                        // rows of this block come from the ranks' dispatch pairs
                        if (!q.live || q.need == 0) return 1;
                        const int* flag = (f.wire_rank ? f.blk_ready : f.blk_cnt) + q.m0 / BM;
                        if (ld_acquire_sys(flag) >= q.need) return 1;
                        if (!block) return 0;
                        const uint64_t t0 = globaltimer_ns();
                        const bool got = wait_flag_ge_sys(flag, q.need, L.status, 600);
                        w_arrive += globaltimer_ns() - t0;
                        return got ? 1 : -1;
                    }
                    if (q.kind == kWorkGemm2) {
                        // the unit's rows of the first GEMM's output: all its column blocks, both CTAs
                        if (ld_acquire_gpu(L.unit_done + q.unit) >= unit_target) return 1;
                        if (!block) return 0;
                        const uint64_t t0 = globaltimer_ns();
                        const bool got = wait_flag_ge_gpu(L.unit_done + q.unit, unit_target, L.status, 601);
                        w_unit += globaltimer_ns() - t0;
                        return got ? 1 : -1;
                    }
                    // weight gradients: their operands are inputs and outputs of the first GEMM of every unit of the
                    // expert; they sit behind all of them in the list, so one check per pair is enough
                    if (q.kind == kWorkWgradGateup && !xperm_ready) {
                        // ... and dW_gateup reads X in slot space, which the gather warps rebuild during the first GEMMs
                        if (L.xperm != nullptr && ld_acquire_gpu(L.expand_done) < L.expand_rows) {
                            if (!block) return 0;
                            const uint64_t t0 = globaltimer_ns();
                            const bool got = wait_flag_ge_gpu(L.expand_done, L.expand_rows, L.status, 603);
                            w_wgrad += globaltimer_ns() - t0;
                            if (!got) return -1;
                        }
                        xperm_ready = true;
                        wgrad_fenced = false;            // one more proxy fence before the first load of X
                    }
                    if (wgrad_ready) return 1;
                    if (ld_acquire_gpu(L.units_complete) >= num_units) { wgrad_ready = true; return 1; }
                    if (!block) return 0;
                    const uint64_t t0 = globaltimer_ns();
                    const bool got = wait_flag_ge_gpu(L.units_complete, num_units, L.status, 602);
                    w_wgrad += globaltimer_ns() - t0;
                    wgrad_ready = got;
                    return got ? 1 : -1;
                };
                auto look_ahead = [&]() -> bool {            // false: a wait ran out
                    const int r = get_item(nxt, false);
                    if (r < 0) return false;
                    if (r == 0) return true;
                    have = true;
                    nxt_ready = false;
                    const int k = item_kind(nxt);
                    if (k >= 0) {
                        ItemGeom qn;
                        item_geometry(L, nxt, rank, qn);
                        nxt_ready = operands_ready(qn, false) == 1;
                    }
                    return true;
                };
                while (ok) {
                    bool cur_ready = false;
                    if (have) {
                        cur = nxt;
                        cur_ready = nxt_ready;
                        have = false;
                    } else if (get_item(cur, true) < 0) {
                        ok = false;
                        break;
                    }
                    const int kind = item_kind(cur);
                    if (kind < 0) break;
                    ItemGeom q;
                    item_geometry(L, cur, rank, q);
                    const LayerPhase& P = L.ph[q.kind];
                    if (!cur_ready && operands_ready(q, true) != 1) { *abort_flag = 1u; ok = false; break; }
                    // generic-proxy stores (peers, other SMs' epilogues) -> async-proxy (TMA) reads; the weight gradients
                    // acquire once, so they need the fence once
                    if (q.kind <= kWorkGemm2 || !wgrad_fenced) fence_proxy_async_all();
                    if (q.kind > kWorkGemm2) wgrad_fenced = true;
                    const int n0 = q.n_blk * BN + (int)rank * (BN / 2);
                    const int look_kb = min(kStagesL - 1, q.nk - 1);   // all stages are in flight: a pause of this thread costs nothing
                    for (int kb = 0; kb < q.nk; ++kb) {
                        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, L.status, 610)) { ok = false; break; }
                        const uint32_t a_dst = smem_base + stage * kStageBytesL;
                        const uint32_t b_dst = a_dst + kAStageBytes;
                        const uint32_t bar = mapa_shared(full_bar(stage), 0);
                        if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * kStageBytesL);
                        else mbar_arrive_cluster(bar);
                        const int k = q.k0 + kb * BK;
                        if (q.kind <= kWorkGemm2) {
                            tma_load_2d_2cta(a_dst, &P.map_a, bar, k, q.m0);
                            if constexpr (!BWD) {
                                tma_load_2d_2cta(b_dst, &P.map_b, bar, k, q.group * P.g.b_group_rows + n0);
                            } else {
                                const int krow = q.group * P.g.b_group_rows + k;
#pragma unroll
                                for (int a = 0; a < BN / 128; ++a) tma_load_2d_2cta(b_dst + a * kAtomBytes, &P.map_b, bar, n0 + 64 * a, krow);
                            }
                        } else {
#pragma unroll
                            for (int a = 0; a < BM / 64; ++a) tma_load_2d_2cta(a_dst + a * kAtomBytes, &P.map_a, bar, q.m0 + 64 * a, k);
#pragma unroll
                            for (int a = 0; a < BN / 128; ++a) tma_load_2d_2cta(b_dst + a * kAtomBytes, &P.map_b, bar, n0 + 64 * a, k);
                        }
                        if (++stage == kStagesL) { stage = 0; phase ^= 1u; }
                        // (the second CTA keeps looking until the first one has published the item)
                        if (kb >= look_kb && !have && (kb == look_kb || rank != 0) && !look_ahead()) { ok = false; break; }
                    }
                }
                if (L.stats != nullptr) {
                    if (w_arrive) atomicAdd(L.stats + kStatWaitArrival, w_arrive);
                    if (w_unit) atomicAdd(L.stats + kStatWaitFirstGemm, w_unit);
                    if (w_wgrad) atomicAdd(L.stats + kStatWaitWgrad, w_wgrad);
                }
            }
        } else if (warp == 1 && rank == 0) {
            // -------------------------------------------------------------- UMMA issuer
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int ss = 0;
            uint32_t sph = 0;
            int iter = 0;
            while (ok) {
                int4 it;
                if (!next_item(ss, sph, 652, it) || it.x < 0) break;
                ItemGeom q;
                item_geometry(L, it, rank, q);
                const bool a_mn = q.kind >= kWorkWgradDown;
                const uint32_t idesc = BWD ? (a_mn ? make_idesc_bf16(2 * BM, BN, true, true) : make_idesc_bf16(2 * BM, BN, false, true))
                                           : make_idesc_bf16(2 * BM, BN, false, false);
                const int as = iter & 1;
                const uint32_t aphase = (iter >> 1) & 1;
                ++iter;
                if (!mbar_wait(tempty_bar(as), aphase ^ 1u, abort_flag, L.status, 620)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(as * BN);
                for (int kb = 0; kb < q.nk; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag, L.status, 621)) { ok = false; break; }
                    tcgen05_fence_after();
                    if (elect_one()) {
                        const uint32_t a_addr = smem_base + stage * kStageBytesL;
                        const uint32_t b_addr = a_addr + kAStageBytes;
#pragma unroll
                        for (int k = 0; k < BK / UK; ++k) {
                            const uint64_t a_desc = a_mn ? make_smem_desc_sw128(a_addr + k * (UK * 128), kAtomBytes, 1024)
                                                         : make_smem_desc_sw128(a_addr + k * (UK * 2), 0, 1024);
                            const uint64_t b_desc = BWD ? make_smem_desc_sw128(b_addr + k * (UK * 128), kAtomBytes, 1024)
                                                        : make_smem_desc_sw128(b_addr + k * (UK * 2), 0, 1024);
                            umma_bf16_ss_2cta(d_tmem, a_desc, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                        }
                        umma_commit_2cta(empty_bar(stage), 3u);
                        if (kb == q.nk - 1) umma_commit_2cta(tfull_bar(as), 3u);
                    }
                    __syncwarp();
                    if (++stage == kStagesL) { stage = 0; phase ^= 1u; }
                }
                if (ok && q.nk == 0) {                       // an expert without rows: the epilogue stores zeros
                    if (elect_one()) umma_commit_2cta(tfull_bar(as), 3u);
                    __syncwarp();
                }
            }
        } else if (warp >= 4) {
            // -------------------------------------------------------------- epilogue / combine / gather
            const int qd = warp & 3;
            const int hh = (warp - 4) >> 2;
            const int r = qd * 32 + lane;
            bool ok = true;
            int ss = 0;
            uint32_t sph = 0;
            int iter = 0;
            int owed = 0;                 // pushed tiles of this warp that are not yet counted as complete
            const uint32_t my_row_smem = push_stage_base + (uint32_t)(warp - 4) * kPushWarpBytes + (uint32_t)lane * kPushRowBytes;
            auto flush_pushes = [&]() {
                if (owed == 0) return;
                tma_store_wait<0>();              // this lane's bulk copies have been written
                fence_proxy_async_all();
                fence_acq_rel_sys();
                __syncwarp();
                if (lane == 0) {
                    const int old = atom_add_acq_rel_gpu(L.push_done, owed);
                    if (old + owed == push_target) signal_ranks();
                }
                owed = 0;
            };
            while (ok) {
                int4 it;
                if (!next_item(ss, sph, 653, it) || it.x < 0) break;
                const bool stamps = L.stats != nullptr && warp == 4 && lane == 0 && rank == 0;
                if (stamps) atomicMax(L.stats + kStatKindFirst + item_kind(it), ~globaltimer_ns());
                ItemGeom q;
                item_geometry(L, it, rank, q);
                const GemmArgs& g = L.ph[q.kind].g;
                if (q.kind >= kWorkWgradDown) flush_pushes();  // count finished pushes before the long tail of weight gradients
                const int as = iter & 1;
                const uint32_t aphase = (iter >> 1) & 1;
                ++iter;
                if (!mbar_wait(tfull_bar(as), aphase, abort_flag, L.status, 630)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t taddr0 = tmem_base + ((uint32_t)(qd * 32) << 16) + (uint32_t)(as * BN + hh * (BN / 2));
                const int n0 = q.n_blk * BN + hh * (BN / 2);
                if (q.kind == kWorkGemm1) {
                    const long row = q.row0 + r;
                    if (q.live) epilogue_thread<BWD ? kEpiDSwiGLU : kEpiSwiGLU>(g, taddr0, row, true, n0, q.n_blk * 2 + hh, false);
                } else if (q.kind == kWorkGemm2) {
                    const long row = q.row0 + r;
                    int src = 0;
                    const unsigned long long dst_row = push_row_address(g, row, q.live, &src);
                    push_epilogue_warp(g, taddr0, dst_row, n0, my_row_smem);
                    if constexpr (BWD) {
                        if (dst_row != 0ull && g.gtw_off != 0ull && q.n_blk == 0 && hh == 0) {
                            float v = 0.f;
                            for (int p = 0; p < g.n_parts_in; ++p) v += __ldcg(g.droute_in + row * g.n_parts_in + p);
                            reinterpret_cast<float*>(g.push_ptrs[src] + g.gtw_off)[g.slot_tk[row]] = v;
                        }
                    }
                    ++owed;
                } else {
                    if constexpr (BWD) {
                        const int m = q.m_in_group + r;
                        const bool row_ok = m < g.m_total;
                        epilogue_thread<kEpiStore>(g, taddr0, row_ok ? q.row0 + r : 0, row_ok, n0, 0, q.nk == 0);
                    }
                }
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(mapa_shared(tempty_bar(as), 0));
                if (stamps) atomicMax(L.stats + kStatKindLast + q.kind, globaltimer_ns());
                if (q.kind == kWorkGemm1) {
                    // this warp's part of the unit's first-GEMM output is stored: count it (the second GEMM and the
                    // weight gradients of this unit wait for all 16 warps of all column blocks)
                    if (lane == 0) {
                        // (the weight gradients wait for one number: how many units are complete)
                        if (atom_add_acq_rel_gpu(L.unit_done + q.unit, 1) == unit_target - 1) red_add_release_gpu(L.units_complete, 1);
                    }
                }
            }
            flush_pushes();
            tma_store_wait<0>();
            if (ok) gather_loop();            // the list is done: help with the landed rows
        } else if (warp >= 2) {
            if (f.wire_rank) replicate_loop();
            if constexpr (BWD) {
                if (L.xperm != nullptr) expand_loop();
            }
            gather_loop();
        }
    }

    tcgen05_fence_before();
    cluster_sync_all();
    if (warp == 2) {
        tcgen05_fence_after();
        tmem_dealloc_2cta(tmem_base, kTmemCols);
    }
}

// -------------------------------------------------------------------------------------------------
// Scheduler: builds the work list (one block).  See the head of this file for the order.
// -------------------------------------------------------------------------------------------------
struct ScheduleArgs {
    const int* unit_order;
    const int* num_units;
    int max_units;
    const int* seg_offsets;
    const int* unit_blk;
    const int* mblock_expert;
    const int* expert_total_local;
    int El;
    int nb1, nb2;              // column blocks of the first / second GEMM
    int bwd;
    int mu_wd, nb_wd;          // weight gradient dW_down: row units and column blocks per expert
    int mu_wg, nb_wg;          // dW_gateup
    int group_units, lag_percent, min_lag_items;
    int T, reduce_chunk;
    int4* work;
    int max_work;
    int* num_work;
    int2* expert_units;
    const int* ok;
};

__global__ void __launch_bounds__(256) layer_schedule_kernel(const ScheduleArgs a) {
    if (a.ok != nullptr && *a.ok == 0) return;
    const int gtid = blockIdx.x * blockDim.x + threadIdx.x, nthreads = gridDim.x * blockDim.x;
    const int U = min(*a.num_units, a.max_units);
    const int SG = max(1, a.group_units);
    const int NG = (U + SG - 1) / SG;
    auto gsize = [&](int g) { return min(SG, U - g * SG); };
    // first / second GEMM items of batch g, tile r: column-block major over the batch's units
    auto emit_gemm = [&](int pos, int kind, int g, int r) {
        const int s = gsize(g);
        const int n_blk = r / s;
        const int u = a.unit_order[g * SG + (r - n_blk * s)];
        const int blk0 = a.unit_blk[u];
        const int two = (a.unit_blk[u + 1] - blk0) == 2 ? 1 : 0;
        const int le = a.mblock_expert[blk0];
        const int valid_end = a.seg_offsets[le] + a.expert_total_local[le];        // rows past it are padding
        const int need0 = max(0, min(128, valid_end - blk0 * 128));
        const int need1 = two ? max(0, min(128, valid_end - (blk0 + 1) * 128)) : 0;
        if (pos < a.max_work) a.work[pos] = make_int4(kind | (two << 4) | (le << 8), u, n_blk | (need0 << 16) | (need1 << 24), blk0);
    };
    // The second GEMM of batch j is placed `lag` first-GEMM items behind the end of batch j's first GEMM: lag_percent of a
    // batch, but at least min_lag_items (about two items per CTA pair, so that the items it waits for have not merely been
    // claimed but are finished when a worker reaches it).  With lg = whole batches of lag and head = the rest:
    //   block B_g = [first `head` items of G1(g)] [G2(g - lg)] [rest of G1(g)],   g = 0 .. NG - 1 + lg
    const int full1 = SG * a.nb1, full2 = SG * a.nb2;
    const int lag_items = max((int)(((long)full1 * a.lag_percent + 99) / 100), a.min_lag_items);
    const int lg = max(1, (lag_items + full1 - 1) / full1);
    const int head_full = min(full1, max(0, lag_items - (lg - 1) * full1));
    // blocks take the schedule's blocks in turn
    for (int g = blockIdx.x; g < NG + lg && NG > 0; g += gridDim.x) {
        const int g2 = g - lg;                                     // batch whose second GEMM sits in this block
        // all batches but the last are full
        const int before1 = g < NG ? g * full1 : U * a.nb1;
        const int c2 = min(max(g2, 0), NG);
        const int before2 = c2 < NG ? c2 * full2 : U * a.nb2;
        const int off = before1 + before2;
        const int n1 = g < NG ? gsize(g) * a.nb1 : 0;
        const int n2 = (g2 >= 0 && g2 < NG) ? gsize(g2) * a.nb2 : 0;
        const int head = min(n1, head_full);
        for (int i = threadIdx.x; i < n1 + n2; i += blockDim.x) {
            if (i < head) emit_gemm(off + i, kWorkGemm1, g, i);
            else if (i < head + n2) emit_gemm(off + i, kWorkGemm2, g2, i - head);
            else emit_gemm(off + i, kWorkGemm1, g, i - n2);
        }
    }
    int pos = U * (a.nb1 + a.nb2);
    if (a.bwd) {
        const int per_wd = a.mu_wd * a.nb_wd, per_wg = a.mu_wg * a.nb_wg;
        for (int i = gtid; i < a.El * per_wd; i += nthreads) {
            const int e = i / per_wd, r = i - e * per_wd;
            const int n_blk = r / a.mu_wd;
            const int k0 = a.seg_offsets[e], nk = (a.seg_offsets[e + 1] - k0) / BK;
            if (pos + i < a.max_work) a.work[pos + i] = make_int4(kWorkWgradDown | (e << 8), k0, n_blk | ((r - n_blk * a.mu_wd) << 16), nk);
        }
        pos += a.El * per_wd;
        for (int i = gtid; i < a.El * per_wg; i += nthreads) {
            const int e = i / per_wg, r = i - e * per_wg;
            const int n_blk = r / a.mu_wg;
            const int k0 = a.seg_offsets[e], nk = (a.seg_offsets[e + 1] - k0) / BK;
            if (pos + i < a.max_work) a.work[pos + i] = make_int4(kWorkWgradGateup | (e << 8), k0, n_blk | ((r - n_blk * a.mu_wg) << 16), nk);
        }
        pos += a.El * per_wg;
    }
    if (gtid == 0) *a.num_work = min(pos, a.max_work);
    // units are numbered expert by expert: first unit and unit count of every expert
    for (int e = gtid; e < a.El; e += nthreads) {
        int first = 0;
        for (int j = 0; j < e; ++j) first += ((a.seg_offsets[j + 1] - a.seg_offsets[j]) / 128 + 1) / 2;
        a.expert_units[e] = make_int2(first, ((a.seg_offsets[e + 1] - a.seg_offsets[e]) / 128 + 1) / 2);
    }
}

template <bool BWD>
cudaError_t launch_layer(const LayerArgs& L, int num_sms, cudaStream_t stream) {
    auto kern = moe_layer_kernel<BWD>;
    static bool configured[64] = {};
    if (cudaError_t e = ensure_smem_limit(kern, kSmemBytesL, configured); e != cudaSuccess) return e;
    int grid = num_sms & ~1;
    if (grid < 2 * (L.f.num_dispatch_clusters + 1)) return cudaErrorInvalidConfiguration;
    // All CTAs must be resident at once (workers wait for rows that dispatch pairs of OTHER ranks send, and this
    // rank's dispatch pairs serve the others): a cooperative launch makes the runtime check that.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytesL;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;
    at[0].val.cooperative = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, L);
}

}  // namespace

int moe_layer_max_work(int bwd, int max_units, int H, int I, int El, int T, int reduce_chunk) {
    const int nbH = (H + BN - 1) / BN, nbI = (I + BN - 1) / BN, nb2I = (2 * I + BN - 1) / BN;
    long n = bwd ? (long)max_units * (nbI + nbH) : (long)max_units * (nb2I + nbH);
    if (bwd) {
        const int mu_wd = (H + 2 * BM - 1) / (2 * BM), mu_wg = (2 * I + 2 * BM - 1) / (2 * BM);
        n += (long)El * (mu_wd * nbI + mu_wg * nbH);
    }
    (void)T; (void)reduce_chunk;
    n += 1;
    return (int)n;
}

cudaError_t moe_layer_schedule(const LayerParams& p, cudaStream_t stream) {
    if (p.reduce_chunk <= 0 || p.group_units <= 0 || p.lag_percent < 0 || p.lag_percent > 100 || p.El <= 0) return cudaErrorInvalidValue;
    const int H = p.H, I = p.I;
    ScheduleArgs a{};
    a.unit_order = p.unit_order; a.num_units = p.lay.num_units_dev; a.max_units = p.lay.max_units;
    a.seg_offsets = p.seg_offsets; a.El = p.El;
    a.unit_blk = p.lay.unit_blk; a.mblock_expert = p.lay.mblock_expert; a.expert_total_local = p.expert_total_local;
    a.nb1 = p.bwd ? (I + BN - 1) / BN : (2 * I + BN - 1) / BN;
    a.nb2 = (H + BN - 1) / BN;
    a.bwd = p.bwd;
    a.mu_wd = (H + 2 * BM - 1) / (2 * BM); a.nb_wd = (I + BN - 1) / BN;
    a.mu_wg = (2 * I + 2 * BM - 1) / (2 * BM); a.nb_wg = (H + BN - 1) / BN;
    a.group_units = p.group_units; a.lag_percent = p.lag_percent;
    a.min_lag_items = p.min_lag_items > 0 ? p.min_lag_items : 0;
    a.T = p.T; a.reduce_chunk = p.reduce_chunk;
    a.work = static_cast<int4*>(p.work); a.max_work = p.max_work; a.num_work = p.num_work;
    a.expert_units = reinterpret_cast<int2*>(p.expert_units);
    a.ok = p.geom_ok;
    layer_schedule_kernel<<<32, 256, 0, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t moe_layer_launch(const LayerParams& p, cudaStream_t stream) {
    if (p.H % BK != 0 || p.I % BK != 0 || p.slot_rows % BM != 0 || p.slot_rows <= 0 || p.out_rows % BM != 0 || p.out_rows <= 0 ||
        p.out_rows > p.slot_rows || p.K > 32 || p.N > 32)
        return cudaErrorInvalidValue;
    if (reinterpret_cast<uintptr_t>(p.f.x) % 16 != 0 || p.f.off_slot_x % 16 != 0 || p.push.landing_off % 16 != 0) return cudaErrorInvalidValue;
    if (p.reduce_chunk <= 0 || p.group_units <= 0 || p.lag_percent < 0 || p.lag_percent > 100) return cudaErrorInvalidValue;
    LayerArgs L{};
    cudaError_t e;
    const int H = p.H, I = p.I, El = p.El;
    const uint64_t S = (uint64_t)p.slot_rows;      // rows of the operand table in the arena
    const uint64_t R = (uint64_t)p.out_rows;       // rows of the tensors this call allocated
    auto base_args = [&](GemmArgs& g) {
        g.max_mblocks = p.out_rows / BM;
        g.num_mblocks_dev = p.lay.num_mblocks_dev;
        g.mblock_expert = p.lay.mblock_expert;
        g.unit_blk = p.lay.unit_blk;
        g.num_units_dev = p.lay.num_units_dev;
        g.max_units = p.lay.max_units;
        g.seg_offsets = p.seg_offsets;
        g.num_groups = El;
        g.status = p.status;
    };
    auto push_args = [&](GemmArgs& g) {
        g.push_ptrs = reinterpret_cast<const unsigned long long*>(p.push.arena_ptrs);
        g.push_off = p.push.landing_off;
        g.slot_tk = p.push.slot_tk;
        g.slot_row = p.push.slot_row;
        g.recv_row_base = p.push.recv_row_base;
        g.num_ranks = p.push.num_ranks;
        g.ldd = H;
    };
    GemmArgs& g1 = L.ph[kWorkGemm1].g;
    GemmArgs& g2 = L.ph[kWorkGemm2].g;
    base_args(g1);
    base_args(g2);
    if (!p.bwd) {
        // gate_up + SwiGLU: A = slot_x [S,H], B = W_gateup [El*2I, H] K-major
        if ((e = make_map(&L.ph[0].map_a, p.slot_x, S, H, BK, BM)) != cudaSuccess) return e;
        if ((e = make_map(&L.ph[0].map_b, p.w1, (uint64_t)El * 2 * I, H, BK, BN / 2)) != cudaSuccess) return e;
        g1.k_total = H; g1.n_total = 2 * I; g1.num_n_blocks = (2 * I + BN - 1) / BN; g1.b_group_rows = 2 * I;
        g1.d = static_cast<__nv_bfloat16*>(p.out0); g1.ldd = I;
        g1.aux = static_cast<__nv_bfloat16*>(p.out1); g1.ld_aux = 2 * I;
        g1.row_w = p.row_w;
        // down + push: A = act [S,I], B = W_down [El*H, I] K-major
        if ((e = make_map(&L.ph[1].map_a, p.out0, R, I, BK, BM)) != cudaSuccess) return e;
        if ((e = make_map(&L.ph[1].map_b, p.w2, (uint64_t)El * H, I, BK, BN / 2)) != cudaSuccess) return e;
        g2.k_total = I; g2.n_total = H; g2.num_n_blocks = (H + BN - 1) / BN; g2.b_group_rows = H;
        push_args(g2);
    } else {
        // grad_act + dSwiGLU: A = slot_x (dY) [S,H], B = W_down [El*H, I] MN-major
        if ((e = make_map(&L.ph[0].map_a, p.slot_x, S, H, BK, BM)) != cudaSuccess) return e;
        if ((e = make_map(&L.ph[0].map_b, p.w1, (uint64_t)El * H, I, 64, BK)) != cudaSuccess) return e;
        g1.k_total = H; g1.n_total = I; g1.num_n_blocks = (I + BN - 1) / BN; g1.b_group_rows = H;
        g1.d = static_cast<__nv_bfloat16*>(p.out0); g1.ldd = I;
        g1.aux = static_cast<__nv_bfloat16*>(p.out1); g1.ld_aux = 2 * I;
        g1.preact = static_cast<const __nv_bfloat16*>(p.preact);
        g1.row_w = p.row_w;
        g1.droute_part = p.droute_part; g1.n_parts = 2 * ((I + BN - 1) / BN);
        // dX + push: A = dGU [S,2I], B = W_gateup [El*2I, H] MN-major
        if ((e = make_map(&L.ph[1].map_a, p.out1, R, 2 * I, BK, BM)) != cudaSuccess) return e;
        if ((e = make_map(&L.ph[1].map_b, p.w2, (uint64_t)El * 2 * I, H, 64, BK)) != cudaSuccess) return e;
        g2.k_total = 2 * I; g2.n_total = H; g2.num_n_blocks = (H + BN - 1) / BN; g2.b_group_rows = 2 * I;
        push_args(g2);
        g2.gtw_off = p.gtw_off; g2.droute_in = p.droute_part; g2.n_parts_in = g1.n_parts;
        // dW_down[e] = dY[seg]^T . act_w[seg]  ([H, I]);  dW_gateup[e] = dGU[seg]^T . X[seg]  ([2I, H])
        GemmArgs& gd = L.ph[kWorkWgradDown].g;
        GemmArgs& gg = L.ph[kWorkWgradGateup].g;
        base_args(gd);
        base_args(gg);
        if ((e = make_map(&L.ph[2].map_a, p.slot_x, S, H, 64, BK)) != cudaSuccess) return e;
        if ((e = make_map(&L.ph[2].map_b, p.out0, R, I, 64, BK)) != cudaSuccess) return e;
        gd.m_total = H; gd.n_total = I; gd.num_n_blocks = (I + BN - 1) / BN; gd.d = static_cast<__nv_bfloat16*>(p.dw_down); gd.ldd = I;
        if ((e = make_map(&L.ph[3].map_a, p.out1, R, 2 * I, 64, BK)) != cudaSuccess) return e;
        if ((e = make_map(&L.ph[3].map_b, p.xperm, R, H, 64, BK)) != cudaSuccess) return e;
        gg.m_total = 2 * I; gg.n_total = H; gg.num_n_blocks = (H + BN - 1) / BN; gg.d = static_cast<__nv_bfloat16*>(p.dw_gateup); gg.ldd = H;
    }
    L.f = p.f;
    L.f.tile_counter = nullptr;
    L.slot_x = static_cast<__nv_bfloat16*>(const_cast<void*>(p.slot_x));
    if (p.f.wire_rank) {
        if (p.f.slot_src == nullptr || p.f.blk_ready == nullptr || p.f.off_slot_src % 4 != 0) return cudaErrorInvalidValue;
        L.f.replicate_counter = p.sync + 6;
    }
    L.work = static_cast<const int4*>(p.work);
    L.num_work = p.num_work;
    L.max_work = p.max_work;
    L.expert_units = reinterpret_cast<const int2*>(p.expert_units);
    L.item_counter = p.sync;
    L.push_done = p.sync + 1;
    L.units_complete = p.sync + 2;
    L.gather_counter = p.sync + 3;
    if (p.bwd && p.x_rows != nullptr) {
        L.x_rows = static_cast<const __nv_bfloat16*>(p.x_rows);
        L.x_slot_row = p.push.slot_row;
        L.xperm = static_cast<__nv_bfloat16*>(const_cast<void*>(p.xperm));
        L.expand_rows = p.expand_rows;
        L.expand_counter = p.sync + 4;
        L.expand_done = p.sync + 5;
    }
    L.unit_done = p.sync + 8;
    L.signal_ptrs = p.signal_ptrs;
    L.my_signal = p.my_signal;
    L.rank = p.rank; L.N = p.N; L.epoch = p.epoch;
    L.landing = static_cast<const __nv_bfloat16*>(p.landing);
    L.out = static_cast<__nv_bfloat16*>(p.out);
    L.gtw_in = p.gtw_in;
    L.gtw_out = p.gtw_out;
    L.stats = p.stats;
    L.geom_ok = p.geom_ok;
    L.status = p.status;

    if ((e = moe_layer_schedule(p, stream)) != cudaSuccess) return e;
    const int sms = default_sms(p.num_sms);
    return p.bwd ? launch_layer<true>(L, sms, stream) : launch_layer<false>(L, sms, stream);
}

}  // namespace tmoe
