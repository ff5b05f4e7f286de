// Routing preparation: everything that turns topk_idx [T,K] into deterministic destinations.
//
//   route_hist      per-chunk histograms over experts, destination ranks and distinct-rank count
//   route_scan      exclusive scan over chunks -> per-source totals; publishes them to every rank
//                   (P2P stores into the peers' metadata table) and crosses a bounded barrier
//   layout_finalize from the all-gathered [ranks, E+ranks+2] table computes, identically on every rank:
//                   padded per-expert segment offsets of every rank's slot space, this source's
//                   offset inside every expert segment, row bases of the token-once receive buffers,
//                   the block->expert map of this rank and the sizes the host needs
//   route_assign    replays the chunks and gives every (token,k) its slot on the destination rank and
//                   every (token, destination rank) its row there
//
// Slots are deterministic: slot = segment offset of the expert + rows of lower source ranks +
// rank of the entry among this source's entries for that expert.  The sender therefore writes each
// token straight to its final place and backward reuses the same places.
//
// Reference counterparts: csrc/kernels/layout.cu:9-149 (per-rank / per-expert counts, is_token_in_rank),
// csrc/kernels/intranode.cu:11-159 (count exchange + prefix matrices) and the receiver-side
// atomicAdd slot claim at csrc/teramoe/teramoe_orchestrator.cu:1238-1259, which this replaces.
#include "routing.h"

#include <cuda_bf16.h>

#include "ptx.cuh"

namespace tmoe {

namespace {

constexpr int kChunkTokens = 128;  // tokens per chunk = threads per block of hist/assign

__device__ __forceinline__ int64_t load_topk(const void* idx, int is64, long i) {
    return is64 ? reinterpret_cast<const int64_t*>(idx)[i] : (int64_t) reinterpret_cast<const int32_t*>(idx)[i];
}

// columns of a histogram row: [0,E) experts, [E,E+N) destination ranks, E+N = sum of distinct ranks, E+N+1 = tokens
__global__ void __launch_bounds__(kChunkTokens)
route_hist_kernel(const void* topk_idx, int is64, int T, int K, int E, int N, int* chunk_hist, uint8_t* in_rank /* [T,N] bool or null */) {
    extern __shared__ int sh[];
    const int C = E + N + 2;
    const int e_local = E / N;
    for (int i = threadIdx.x; i < C; i += blockDim.x) sh[i] = 0;
    __syncthreads();
    const int t = blockIdx.x * kChunkTokens + threadIdx.x;
    if (t < T) {
        uint32_t mask = 0;
        for (int k = 0; k < K; ++k) {
            const int64_t e = load_topk(topk_idx, is64, (long)t * K + k);
            if (e >= 0 && e < E) {
                atomicAdd(&sh[(int)e], 1);
                mask |= 1u << ((int)e / e_local);
            }
        }
        for (int d = 0; d < N; ++d) {
            if (mask >> d & 1u) atomicAdd(&sh[E + d], 1);
            if (in_rank != nullptr) in_rank[(long)t * N + d] = (uint8_t)(mask >> d & 1u);   // is_token_in_rank of the layout API
        }
        atomicAdd(&sh[E + N], __popc(mask));
        atomicAdd(&sh[E + N + 1], 1);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < C; i += blockDim.x) chunk_hist[(long)blockIdx.x * C + i] = sh[i];
}

// Column sums of the per-chunk histograms: the counts of get_dispatch_layout.
__global__ void __launch_bounds__(256) route_sum_kernel(const int* chunk_hist, int num_chunks, int C, int* totals) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    int s = 0;
    for (int ch = 0; ch < num_chunks; ++ch) s += chunk_hist[(long)ch * C + c];
    totals[c] = s;
}

// One block.  chunk_base[chunk][c] = exclusive prefix over chunks; totals go to row `rank` of the
// metadata table of every peer; then a barrier over all ranks (skipped when epoch == 0, which the
// single-device emulation of several ranks uses).
__global__ void __launch_bounds__(1024)
route_scan_kernel(const int* chunk_hist, int* chunk_base, int num_chunks, int C, int rank, int N,
                  const uint64_t* meta_ptrs /* [N] address of each rank's table [N][C] */,
                  const uint64_t* signal_ptrs /* [N] address of each rank's int[N] signal row */, int epoch, int* status) {
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        int run = 0;
#pragma unroll 8
        for (int ch = 0; ch < num_chunks; ++ch) {
            const int v = chunk_hist[(long)ch * C + c];
            chunk_base[(long)ch * C + c] = run;
            run += v;
        }
        for (int d = 0; d < N; ++d) reinterpret_cast<int*>(meta_ptrs[d])[(long)rank * C + c] = run;
    }
    if (epoch == 0) return;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < N) {
        int* peer_sig = reinterpret_cast<int*>(signal_ptrs[threadIdx.x]);
        st_release_sys(peer_sig + rank, epoch);
        const int* my_sig = reinterpret_cast<const int*>(signal_ptrs[rank]);
        if (!wait_flag_ge_sys(my_sig + threadIdx.x, epoch, status, 400 + threadIdx.x)) return;
    }
}

__global__ void __launch_bounds__(1024)
layout_finalize_kernel(const int* meta /* [N][C] */, int rank, int N, int E, LayoutOut o, int cap_rows, int cap_slots, int cap_tokens) {
    const int C = E + N + 2;
    const int e_local = E / N;
    __shared__ int sh_spad[64];
    __shared__ int sh_rows[64];
    // per-expert totals and this source's offset inside every expert segment
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int tot = 0, before = 0;
        for (int s = 0; s < N; ++s) {
            const int v = meta[s * C + e];
            if (s < rank) before += v;
            tot += v;
        }
        o.expert_total[e] = tot;
        o.my_src_off[e] = before;
    }
    __syncthreads();
    // padded segment offsets inside every rank's slot space; row bases of every rank's receive buffer
    if (threadIdx.x < N) {
        const int d = threadIdx.x;
        int run = 0;
        for (int le = 0; le < e_local; ++le) {
            const int e = d * e_local + le;
            o.seg_off_all[e] = run;
            run += (o.expert_total[e] + 127) / 128 * 128;
        }
        sh_spad[d] = run;
        int rows = 0;
        for (int s = 0; s < N; ++s) {
            if (s == rank) o.my_row_base[d] = rows;
            if (d == rank) o.recv_row_base[s] = rows;
            rows += meta[s * C + E + d];
        }
        if (d == rank) o.recv_row_base[N] = rows;
        sh_rows[d] = rows;
    }
    __syncthreads();
    const int my_spad = sh_spad[rank];
    if (threadIdx.x == 0) {
        int rmax = 0, smax = 0, lmax = 0, tmax = 0;
        for (int d = 0; d < N; ++d) {
            rmax = max(rmax, sh_rows[d]);
            smax = max(smax, sh_spad[d]);
            lmax = max(lmax, meta[d * C + E + N]);
            tmax = max(tmax, meta[d * C + E + N + 1]);
        }
        o.sizes[0] = sh_rows[rank];          // rows received by this rank (token-once)
        o.sizes[1] = my_spad;                // padded slots of this rank
        o.sizes[2] = meta[rank * C + E + N]; // combine landing rows of this rank
        o.sizes[3] = rmax;
        o.sizes[4] = smax;
        o.sizes[5] = lmax;
        o.sizes[6] = my_spad / 128;
        o.sizes[7] = tmax;
        // capacities the caller sized its tables with before it knew these numbers (0: it waits for them instead);
        // every rank sees the same maxima, so every rank gets the same answer
        o.sizes[8] = (cap_rows <= 0 || (rmax <= cap_rows && smax <= cap_slots && tmax <= cap_tokens)) ? 1 : 0;
        o.num_mblocks[0] = my_spad / 128;
        o.seg_offsets[e_local] = my_spad;
        // send order of a fused dispatch: destination ranks in rotation starting with this rank
        int run = 0;
        for (int p = 0; p < N; ++p) {
            const int d = (rank + p) % N;
            for (int le = 0; le < e_local; ++le) {
                const int e = d * e_local + le;
                o.send_base[e] = run;
                run += meta[rank * C + e];
            }
        }
        o.num_mblocks[1] = run;
    }
    // this rank's segment table
    for (int le = threadIdx.x; le < e_local; le += blockDim.x) o.seg_offsets[le] = o.seg_off_all[rank * e_local + le];
}

// Pad slots of this rank's segments (row -1, weight 0), the block->expert map and the unit table of
// the CTA-pair GEMMs (a unit = one or two consecutive 128-row blocks of one expert; unit_blk[u] is
// its first block, unit_blk[num_units] the block count).  Runs after the host has placed the slot
// tables (their offsets depend on the sizes computed by layout_finalize).
__global__ void __launch_bounds__(256)
slot_pad_fill_kernel(const int* seg_offsets, const int* expert_total_local, int e_local, int* slot_row, float* slot_w, int* slot_tk,
                     int* mblock_expert, int* unit_blk, int* num_units, const int* ok) {
    __shared__ int unit_base;
    if (ok != nullptr && *ok == 0) return;       // the layout does not fit the tables: the caller repeats the call
    for (int le = blockIdx.x; le < e_local; le += gridDim.x) {
        const int first = seg_offsets[le] + expert_total_local[le];
        const int last = seg_offsets[le + 1];
        const int blk0 = seg_offsets[le] / 128, blk1 = last / 128;
        for (int b = blk0 + threadIdx.x; b < blk1; b += blockDim.x) mblock_expert[b] = le;
        for (int s = first + threadIdx.x; s < last; s += blockDim.x) {
            slot_row[s] = -1;
            slot_w[s] = 0.f;
            slot_tk[s] = -1;
        }
        if (unit_blk != nullptr) {
            __syncthreads();
            if (threadIdx.x == 0) {
                int base = 0;
                for (int j = 0; j < le; ++j) base += ((seg_offsets[j + 1] - seg_offsets[j]) / 128 + 1) / 2;
                unit_base = base;
            }
            __syncthreads();
            const int nu = (blk1 - blk0 + 1) / 2;
            for (int i = threadIdx.x; i < nu; i += blockDim.x) unit_blk[unit_base + i] = blk0 + 2 * i;
            if (le == e_local - 1 && threadIdx.x == 0) {
                unit_blk[unit_base + nu] = blk1;
                num_units[0] = unit_base + nu;
            }
        }
    }
}

// One block per chunk, one thread per token; warps take turns so that ranks inside a chunk follow
// (warp, k, lane) order.  run[] lives in shared memory and starts from the chunk's scanned base.
__global__ void __launch_bounds__(kChunkTokens)
route_assign_kernel(const void* topk_idx, int is64, int T, int K, int E, int N, const int* chunk_base, LayoutOut o,
                    int* send_slot /* [T,K] */, int* send_row /* [T,N] */, int* land_off /* [T] */, int* ndst /* [T] */,
                    int* send_order /* [T*K] or null */) {
    extern __shared__ int run[];
    const int C = E + N + 2;
    const int e_local = E / N;
    for (int i = threadIdx.x; i < C; i += blockDim.x) run[i] = chunk_base[(long)blockIdx.x * C + i];
    __syncthreads();
    const int t = blockIdx.x * kChunkTokens + threadIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t lt = (1u << lane) - 1u;
    for (int w = 0; w < kChunkTokens / 32; ++w) {
        if (warp == w) {
            uint32_t mask = 0;
            for (int k = 0; k < K; ++k) {
                int64_t e64 = (t < T) ? load_topk(topk_idx, is64, (long)t * K + k) : -1;
                const int e = (e64 >= 0 && e64 < E) ? (int)e64 : -1;
                const uint32_t same = __match_any_sync(0xffffffffu, e);
                int slot = -1;
                if (e >= 0) {
                    const int base = run[e];
                    const int j = base + __popc(same & lt);
                    slot = o.seg_off_all[e] + o.my_src_off[e] + j;
                    mask |= 1u << (e / e_local);
                    if (send_order != nullptr) send_order[o.send_base[e] + j] = t * K + k;
                }
                __syncwarp();
                if (e >= 0 && (same & lt) == 0) run[e] += __popc(same);
                __syncwarp();
                if (t < T) send_slot[(long)t * K + k] = slot;
            }
            for (int d = 0; d < N; ++d) {
                const bool hit = (mask >> d) & 1u;
                const uint32_t b = __ballot_sync(0xffffffffu, hit);
                const int base = run[E + d];
                if (t < T) send_row[(long)t * N + d] = hit ? o.my_row_base[d] + base + __popc(b & lt) : -1;
                __syncwarp();
                if (lane == 0) run[E + d] = base + __popc(b);
                __syncwarp();
            }
            // exclusive scan of distinct-rank counts inside the warp
            const int n = __popc(mask);
            int incl = n;
            for (int s = 1; s < 32; s <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, s);
                if (lane >= s) incl += v;
            }
            const int base = run[E + N];
            if (t < T) {
                land_off[t] = base + incl - n;
                ndst[t] = n;
            }
            __syncwarp();
            if (lane == 31) run[E + N] = base + incl;
        }
        __syncthreads();
    }
}

}  // namespace

int route_chunk_tokens() { return kChunkTokens; }

cudaError_t route_hist(const void* topk_idx, int is64, int T, int K, int E, int N, int* chunk_hist, uint8_t* in_rank, cudaStream_t stream) {
    const int chunks = (T + kChunkTokens - 1) / kChunkTokens;
    if (chunks == 0) return cudaSuccess;
    route_hist_kernel<<<chunks, kChunkTokens, (E + N + 2) * sizeof(int), stream>>>(topk_idx, is64, T, K, E, N, chunk_hist, in_rank);
    return cudaGetLastError();
}

cudaError_t route_sum(const int* chunk_hist, int num_chunks, int C, int* totals, cudaStream_t stream) {
    route_sum_kernel<<<(C + 255) / 256, 256, 0, stream>>>(chunk_hist, num_chunks, C, totals);
    return cudaGetLastError();
}

cudaError_t route_scan(const int* chunk_hist, int* chunk_base, int num_chunks, int E, int rank, int N, const uint64_t* meta_ptrs,
                       const uint64_t* signal_ptrs, int epoch, int* status, cudaStream_t stream) {
    route_scan_kernel<<<1, 1024, 0, stream>>>(chunk_hist, chunk_base, num_chunks, E + N + 2, rank, N, meta_ptrs, signal_ptrs, epoch,
                                              status);
    return cudaGetLastError();
}

cudaError_t layout_finalize(const int* meta, int rank, int N, int E, const LayoutOut& out, int cap_rows, int cap_slots, int cap_tokens,
                            cudaStream_t stream) {
    if (N > 64) return cudaErrorInvalidValue;
    layout_finalize_kernel<<<1, 1024, 0, stream>>>(meta, rank, N, E, out, cap_rows, cap_slots, cap_tokens);
    return cudaGetLastError();
}

cudaError_t slot_pad_fill(const int* seg_offsets, const int* expert_total_local, int e_local, int* slot_row, float* slot_w,
                          int* slot_tk, int* mblock_expert, int* unit_blk, int* num_units, const int* ok, cudaStream_t stream) {
    if (e_local <= 0) return cudaSuccess;
    slot_pad_fill_kernel<<<e_local < 256 ? e_local : 256, 256, 0, stream>>>(seg_offsets, expert_total_local, e_local, slot_row, slot_w,
                                                                            slot_tk, mblock_expert, unit_blk, num_units, ok);
    return cudaGetLastError();
}

cudaError_t route_assign(const void* topk_idx, int is64, int T, int K, int E, int N, const int* chunk_base, const LayoutOut& out,
                         int* send_slot, int* send_row, int* land_off, int* ndst, int* send_order, cudaStream_t stream) {
    const int chunks = (T + kChunkTokens - 1) / kChunkTokens;
    if (chunks == 0) return cudaSuccess;
    route_assign_kernel<<<chunks, kChunkTokens, (E + N + 2) * sizeof(int), stream>>>(topk_idx, is64, T, K, E, N, chunk_base, out,
                                                                                  send_slot, send_row, land_off, ndst, send_order);
    return cudaGetLastError();
}

namespace {
// One block.  Per 128-row block: the arrival group of the latest source that owns rows in it (source s
// reaches this rank in phase (rank - s) mod N of its rotation; phases are binned into `groups`); then
// the units sorted by group.
__global__ void __launch_bounds__(256)
arrival_order_kernel(const int* meta, int rank, int N, int E, int groups, const int* seg_offsets, const int* unit_blk,
                     const int* num_units_p, int max_units, int* blk_group, int* unit_order, const int* ok) {
    if (ok != nullptr && *ok == 0) return;
    const int C = E + N + 2;
    const int e_local = E / N;
    for (int le = threadIdx.x; le < e_local; le += blockDim.x) {
        const int e = rank * e_local + le;
        const int b0 = seg_offsets[le] / 128, b1 = seg_offsets[le + 1] / 128;
        for (int b = b0; b < b1; ++b) {
            const int lo = (b - b0) * 128, hi = lo + 128;
            int cum = 0, grp = 0;
            for (int s = 0; s < N; ++s) {
                const int c = meta[s * C + e];
                if (c > 0 && cum < hi && cum + c > lo) {
                    const int phase = (rank - s + N) % N;
                    grp = max(grp, phase * groups / N);
                }
                cum += c;
            }
            blk_group[b] = grp;
        }
    }
    __syncthreads();
    // units sorted by group, stable: one ordered compaction pass over the units per group (ballots + warp offsets)
    __shared__ int warp_cnt[8];
    __shared__ int base;
    const int nu = min(num_units_p[0], max_units);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) base = 0;
    __syncthreads();
    for (int gsel = 0; gsel < groups; ++gsel) {
        for (int start = 0; start < nu; start += blockDim.x) {
            const int u = start + threadIdx.x;
            bool match = false;
            if (u < nu) {
                const int b = unit_blk[u];
                int gu = blk_group[b];
                if (unit_blk[u + 1] - b == 2) gu = max(gu, blk_group[b + 1]);
                match = gu == gsel;
            }
            const uint32_t bal = __ballot_sync(0xffffffffu, match);
            if (lane == 0) warp_cnt[warp] = __popc(bal);
            __syncthreads();
            int off = base;
            for (int w2 = 0; w2 < warp; ++w2) off += warp_cnt[w2];
            if (match) unit_order[off + __popc(bal & ((1u << lane) - 1u))] = u;
            __syncthreads();
            if (threadIdx.x == 0) {
                int tot = 0;
                for (int w2 = 0; w2 < (int)(blockDim.x >> 5); ++w2) tot += warp_cnt[w2];
                base += tot;
            }
            __syncthreads();
        }
    }
}
}  // namespace

namespace {
// Pad rows of the slot-space operand table must read as zeros (they take part in the weight gradients).
__global__ void __launch_bounds__(256)
zero_pad_rows_kernel(const int* seg_offsets, const int* expert_total_local, int e_local, __nv_bfloat16* slot_x, int H, const int* ok) {
    if (ok != nullptr && *ok == 0) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int le = blockIdx.x; le < e_local; le += gridDim.x) {
        const int first = seg_offsets[le] + expert_total_local[le];
        const int last = seg_offsets[le + 1];
        for (int s = first + warp; s < last; s += blockDim.x / 32) {
            int4* row = reinterpret_cast<int4*>(slot_x + (long)s * H);
            for (int i = lane; i < H / 8; i += 32) row[i] = make_int4(0, 0, 0, 0);
        }
    }
}
}  // namespace

cudaError_t zero_pad_rows(const int* seg_offsets, const int* expert_total_local, int e_local, void* slot_x, int H, const int* ok,
                          cudaStream_t stream) {
    if (e_local <= 0) return cudaSuccess;
    zero_pad_rows_kernel<<<e_local < 512 ? e_local : 512, 256, 0, stream>>>(seg_offsets, expert_total_local, e_local,
                                                                            static_cast<__nv_bfloat16*>(slot_x), H, ok);
    return cudaGetLastError();
}

cudaError_t arrival_order(const int* meta, int rank, int N, int E, int groups, const int* seg_offsets, const int* unit_blk,
                          const int* num_units, int max_units, int* blk_group, int* unit_order, const int* ok, cudaStream_t stream) {
    arrival_order_kernel<<<1, 256, 0, stream>>>(meta, rank, N, E, groups, seg_offsets, unit_blk, num_units, max_units, blk_group,
                                                unit_order, ok);
    return cudaGetLastError();
}

}  // namespace tmoe
