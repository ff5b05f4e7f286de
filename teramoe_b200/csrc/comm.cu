// Push-model expert-parallel data movement over NVLink peer mappings, plus the local row kernels.
//
//   ep_barrier      bounded all-rank barrier on monotonically increasing epochs
//   dispatch_push   every token row is stored ONCE per destination rank, straight into its final row
//                   of that rank's receive buffer; per-slot and per-row tables are stored with it
//   expand_rows     slot space <- receive rows (row gather; pad slots become zero rows)
//   combine_push    per received token: fp32 sum of its local expert outputs, one bf16 row stored
//                   into the source rank's landing buffer (+ route-weight gradients in backward)
//   combine_reduce  per local token: fp32 sum of the landed rows -> bf16 output row
//   numerics_check  max-abs / cosine / calc_diff statistics of two tensors in one pass
//
// Only stores cross NVLink; no kernel reads a peer's memory.  There are no rings, heads or tails:
// destinations are final, so the only synchronisation is the barrier between phases.
//
// Reference counterparts: csrc/kernels/intranode.cu:197-532 (dispatch), :691-1032 (combine),
// csrc/kernels/utils.cuh:501-531 (barrier_block), csrc/teramoe/teramoe_orchestrator.cu:2849-2976
// (gather role), csrc/kernels/internode_common.cuh:80-240 (combine_token), tests/utils.py:39-43
// (calc_diff).
#include "comm.h"

#include <cuda_bf16.h>

#include "ptx.cuh"

namespace tmoe {

namespace {

// mode 0: signal every rank, then wait for every rank (a barrier); 1: signal only; 2: wait only.
__global__ void ep_barrier_kernel(const uint64_t* signal_ptrs, int rank, int N, int epoch, int* status, int site, uint64_t limit_ns,
                                  int mode, const int* mask) {
    __threadfence_system();
    // ranks marked in `mask` (elastic shrink) are neither signalled nor waited for
    if ((int)threadIdx.x < N && (mask == nullptr || mask[threadIdx.x] == 0)) {
        if (mode != 2) {
            int* peer_sig = reinterpret_cast<int*>(signal_ptrs[threadIdx.x]);
            st_release_sys(peer_sig + rank, epoch);
        }
        if (mode != 1) {
            const int* my_sig = reinterpret_cast<const int*>(signal_ptrs[rank]);
            // A peer that never arrives makes this wait run out: the status block then names the site
            // (site + peer rank) and the kernel returns normally, so the context stays usable.
            wait_flag_ge_sys(my_sig + threadIdx.x, epoch, status, site + threadIdx.x, limit_ns);
        }
    }
}

__device__ __forceinline__ int64_t load_topk(const void* idx, int is64, long i) {
    return is64 ? reinterpret_cast<const int64_t*>(idx)[i] : (int64_t) reinterpret_cast<const int32_t*>(idx)[i];
}

__global__ void __launch_bounds__(256)
dispatch_push_kernel(const __nv_bfloat16* x, const void* topk_idx, int is64, const float* topk_w, int T, int K, int H, int E,
                     int N, const int* send_slot, const int* send_row, const int* land_off, const uint64_t* arena_ptrs,
                     SymOffsets so, int with_meta, const int* ok) {
    if (ok != nullptr && *ok == 0) return;       // the layout does not fit the receivers' tables (fixed-shape mode): send nothing
    const int lane = threadIdx.x & 31;
    const int warps_per_grid = (gridDim.x * blockDim.x) >> 5;
    const int e_local = E / N;
    const int nvec = H / 8;
    for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps_per_grid) {
        const int my_row = (lane < N) ? send_row[(long)t * N + lane] : -1;
        const uint32_t mask = __ballot_sync(0xffffffffu, my_row >= 0);
        const int4* src = reinterpret_cast<const int4*>(x + (long)t * H);
        for (uint32_t m = mask; m != 0; m &= m - 1) {
            const int d = __ffs(m) - 1;
            const int row = __shfl_sync(0xffffffffu, my_row, d);
            int4* dst = reinterpret_cast<int4*>(arena_ptrs[d] + so.recv_x + (uint64_t)row * H * 2);
            warp_copy_row(dst, src, nvec, lane);
        }
        if (with_meta) {
            // per-slot tables: lane k owns entry (t,k)
            int slot = -1, d_of_k = 0;
            if (lane < K) {
                const int64_t e = load_topk(topk_idx, is64, (long)t * K + lane);
                if (e >= 0 && e < E) {
                    slot = send_slot[(long)t * K + lane];
                    d_of_k = (int)e / e_local;
                }
            }
            const int row_of_k = __shfl_sync(0xffffffffu, my_row, d_of_k);
            if (slot >= 0) {
                const uint64_t base = arena_ptrs[d_of_k];
                reinterpret_cast<int*>(base + so.slot_row)[slot] = row_of_k;
                reinterpret_cast<float*>(base + so.slot_w)[slot] = topk_w[(long)t * K + lane];
                reinterpret_cast<int*>(base + so.slot_tk)[slot] = t * K + lane;
            }
            // per-row tables: lane d owns (t, destination d)
            const int lo = land_off[t];
            int j = 0;
            for (int k = 0; k < K; ++k) {
                const int s_k = __shfl_sync(0xffffffffu, slot, k);
                const int d_k = __shfl_sync(0xffffffffu, d_of_k, k);
                if (my_row >= 0 && s_k >= 0 && d_k == lane) {
                    reinterpret_cast<int*>(arena_ptrs[lane] + so.row_slots)[(long)my_row * K + j] = s_k;
                    ++j;
                }
            }
            if (my_row >= 0) {
                int* rs = reinterpret_cast<int*>(arena_ptrs[lane] + so.row_slots) + (long)my_row * K;
                for (int jj = j; jj < K; ++jj) rs[jj] = -1;
            }
            if (my_row >= 0) {
                const uint64_t base = arena_ptrs[lane];
                reinterpret_cast<int*>(base + so.row_tok)[my_row] = t;
                reinterpret_cast<int*>(base + so.row_land)[my_row] = lo + __popc(mask & ((1u << lane) - 1u));
            }
            // what the receiver hands out as recv_topk_idx / recv_topk_weights: lane k writes entry k of the token's row on
            // every rank the token goes to (local expert id and weight where the entry's expert lives there, -1 / 0 elsewhere)
            {
                int64_t e_k = -1;
                float w_k = 0.f;
                if (lane < K) {
                    e_k = load_topk(topk_idx, is64, (long)t * K + lane);
                    if (e_k < 0 || e_k >= E) e_k = -1;
                    else w_k = topk_w[(long)t * K + lane];
                }
                for (uint32_t m = mask; m != 0; m &= m - 1) {
                    const int d = __ffs(m) - 1;
                    const int row = __shfl_sync(0xffffffffu, my_row, d);
                    if (lane < K) {
                        const bool here = e_k >= 0 && (int)e_k / e_local == d;
                        reinterpret_cast<int64_t*>(arena_ptrs[d] + so.row_topk_idx)[(long)row * K + lane] = here ? e_k - (int64_t)d * e_local : -1;
                        reinterpret_cast<float*>(arena_ptrs[d] + so.row_topk_w)[(long)row * K + lane] = here ? w_k : 0.f;
                    }
                }
            }
        }
    }
}

__global__ void __launch_bounds__(256)
expand_rows_kernel(const __nv_bfloat16* rows, const int* slot_row, __nv_bfloat16* out, int num_slots, int H) {
    const int lane = threadIdx.x & 31;
    const int warps_per_grid = (gridDim.x * blockDim.x) >> 5;
    const int nvec = H / 8;
    for (int s = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; s < num_slots; s += warps_per_grid) {
        const int r = slot_row[s];
        int4* dst = reinterpret_cast<int4*>(out + (long)s * H);
        if (r >= 0) {
            const int4* src = reinterpret_cast<const int4*>(rows + (long)r * H);
            warp_copy_row(dst, src, nvec, lane);
        } else {
            for (int i = lane; i < nvec; i += 32) dst[i] = make_int4(0, 0, 0, 0);
        }
    }
}

__device__ __forceinline__ void accum_bf16x8(float (&acc)[8], const int4& v) {
    const uint32_t u[4] = {(uint32_t)v.x, (uint32_t)v.y, (uint32_t)v.z, (uint32_t)v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = unpack_bf16x2(u[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
    }
}
__device__ __forceinline__ int4 pack_bf16x8(const float (&acc)[8]) {
    return make_int4((int)pack_bf16x2(acc[0], acc[1]), (int)pack_bf16x2(acc[2], acc[3]), (int)pack_bf16x2(acc[4], acc[5]),
                     (int)pack_bf16x2(acc[6], acc[7]));
}

__global__ void __launch_bounds__(256)
combine_push_kernel(const __nv_bfloat16* y, const int* row_slots, const int* row_land, const int* recv_row_base, int R, int K,
                    int H, int N, const uint64_t* arena_ptrs, SymOffsets so, const float* droute_part, int n_parts,
                    const int* slot_tk, int with_payload) {
    const int lane = threadIdx.x & 31;
    const int warps_per_grid = (gridDim.x * blockDim.x) >> 5;
    const int nvec = H / 8;
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < R; r += warps_per_grid) {
        int src = 0;
        while (src + 1 < N && r >= recv_row_base[src + 1]) ++src;
        const int my_slot = (lane < K) ? row_slots[(long)r * K + lane] : -1;
        const int nsl = __popc(__ballot_sync(0xffffffffu, my_slot >= 0));
        const uint64_t base = arena_ptrs[src];
        int4* dst = reinterpret_cast<int4*>(base + so.landing + (uint64_t)row_land[r] * H * 2);
        if (!with_payload) {
        } else if (nsl == 1) {
            const int s0 = __shfl_sync(0xffffffffu, my_slot, 0);
            const int4* p = reinterpret_cast<const int4*>(y + (long)s0 * H);
            warp_copy_row(dst, p, nvec, lane);
        } else {
            int i = lane;
            for (; i + 32 < nvec; i += 64) {        // two vectors per lane in flight for every source row
                float acc0[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                float acc1[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                for (int j = 0; j < nsl; ++j) {
                    const int sj = __shfl_sync(0xffffffffu, my_slot, j);
                    const int4* row = reinterpret_cast<const int4*>(y + (long)sj * H);
                    const int4 v0 = row[i], v1 = row[i + 32];
                    accum_bf16x8(acc0, v0);
                    accum_bf16x8(acc1, v1);
                }
                st_na_v4(dst + i, pack_bf16x8(acc0));
                st_na_v4(dst + i + 32, pack_bf16x8(acc1));
            }
            for (; i < nvec; i += 32) {
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                for (int j = 0; j < nsl; ++j) {
                    const int sj = __shfl_sync(0xffffffffu, my_slot, j);
                    accum_bf16x8(acc, reinterpret_cast<const int4*>(y + (long)sj * H)[i]);
                }
                st_na_v4(dst + i, pack_bf16x8(acc));
            }
        }
        if (droute_part != nullptr && my_slot >= 0) {
            float v = 0.f;
            for (int p = 0; p < n_parts; ++p) v += droute_part[(long)my_slot * n_parts + p];
            reinterpret_cast<float*>(base + so.gtw)[slot_tk[my_slot]] = v;
        }
    }
}

__global__ void __launch_bounds__(256)
combine_reduce_kernel(const __nv_bfloat16* landing, const int* land_off, const int* ndst, __nv_bfloat16* out, int T, int H) {
    const int lane = threadIdx.x & 31;
    const int warps_per_grid = (gridDim.x * blockDim.x) >> 5;
    const int nvec = H / 8;
    for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps_per_grid) {
        const int n = ndst[t];
        const long lo = land_off[t];
        int4* dst = reinterpret_cast<int4*>(out + (long)t * H);
        if (n == 1) {
            const int4* p = reinterpret_cast<const int4*>(landing + lo * H);
            for (int i = lane; i < nvec; i += 32) dst[i] = ld_nc_v4(p + i);
        } else {
            for (int i = lane; i < nvec; i += 32) {
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                for (int j = 0; j < n; ++j) accum_bf16x8(acc, ld_nc_v4(reinterpret_cast<const int4*>(landing + (lo + j) * H) + i));
                dst[i] = pack_bf16x8(acc);
            }
        }
    }
}

// Fixed-shape dispatch outputs: rows past the received count (a device scalar) read as "nothing": zero payload,
// expert id -1, weight 0.  One warp per row.
__global__ void __launch_bounds__(256)
tail_fill_kernel(__nv_bfloat16* x, int64_t* idx, float* w, const int* rows_dev, int total_rows, int H, int K) {
    const int lane = threadIdx.x & 31;
    const int warps_per_grid = (gridDim.x * blockDim.x) >> 5;
    const int first = max(0, min(*rows_dev, total_rows));
    for (int r = first + ((blockIdx.x * blockDim.x + threadIdx.x) >> 5); r < total_rows; r += warps_per_grid) {
        int4* row = reinterpret_cast<int4*>(x + (long)r * H);
        for (int i = lane; i < H / 8; i += 32) row[i] = make_int4(0, 0, 0, 0);
        if (lane < K) {
            idx[(long)r * K + lane] = -1;
            w[(long)r * K + lane] = 0.f;
        }
    }
}

// One row per slot goes to the rank that owns the token: landing[slot_tk[s]] on the source of slot s.
__global__ void __launch_bounds__(256)
slot_rows_push_kernel(const __nv_bfloat16* y, const int* slot_tk, const int* slot_row, const int* recv_row_base, int S, int H, int N,
                      const uint64_t* arena_ptrs, uint64_t landing_off) {
    const int lane = threadIdx.x & 31;
    const int warps_per_grid = (gridDim.x * blockDim.x) >> 5;
    const int nvec = H / 8;
    for (int s = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; s < S; s += warps_per_grid) {
        const int tk = slot_tk[s];
        if (tk < 0) continue;
        const int rr = slot_row[s];
        int src = 0;
        while (src + 1 < N && rr >= recv_row_base[src + 1]) ++src;
        int4* dst = reinterpret_cast<int4*>(arena_ptrs[src] + landing_off + (uint64_t)tk * H * 2);
        const int4* p = reinterpret_cast<const int4*>(y + (long)s * H);
        warp_copy_row(dst, p, nvec, lane);
    }
}

// Per-(token,k) landing table [T*K, H]: out[t] = fp32 sum over the token's valid entries (optionally
// weighted by w[t,k]), one rounding.
__global__ void __launch_bounds__(256)
combine_reduce_slots_kernel(const __nv_bfloat16* landing, const void* topk_idx, int is64, __nv_bfloat16* out, int T, int K, int H,
                            int E, const float* weights) {
    const int lane = threadIdx.x & 31;
    const int warps_per_grid = (gridDim.x * blockDim.x) >> 5;
    const int nvec = H / 8;
    for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps_per_grid) {
        int64_t e = -1;
        if (lane < K) e = load_topk(topk_idx, is64, (long)t * K + lane);
        const uint32_t valid = __ballot_sync(0xffffffffu, e >= 0 && e < E);
        int4* dst = reinterpret_cast<int4*>(out + (long)t * H);
        if (weights == nullptr) {
            int i = lane;
            for (; i + 32 < nvec; i += 64) {    // two vectors per lane and entry in flight
                float a0[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                float a1[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                for (uint32_t m = valid; m != 0; m &= m - 1) {
                    const int k = __ffs(m) - 1;
                    const int4* row = reinterpret_cast<const int4*>(landing + ((long)t * K + k) * H);
                    const int4 v0 = ld_nc_v4(row + i), v1 = ld_nc_v4(row + i + 32);
                    accum_bf16x8(a0, v0);
                    accum_bf16x8(a1, v1);
                }
                dst[i] = pack_bf16x8(a0);
                dst[i + 32] = pack_bf16x8(a1);
            }
            for (; i < nvec; i += 32) {
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                for (uint32_t m = valid; m != 0; m &= m - 1) {
                    const int k = __ffs(m) - 1;
                    accum_bf16x8(acc, ld_nc_v4(reinterpret_cast<const int4*>(landing + ((long)t * K + k) * H) + i));
                }
                dst[i] = pack_bf16x8(acc);
            }
            continue;
        }
        for (int i = lane; i < nvec; i += 32) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (uint32_t m = valid; m != 0; m &= m - 1) {
                const int k = __ffs(m) - 1;
                const int4 v = ld_nc_v4(reinterpret_cast<const int4*>(landing + ((long)t * K + k) * H) + i);
                float one[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                accum_bf16x8(one, v);
                const float wk = weights[(long)t * K + k];
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] += wk * one[j];
            }
            dst[i] = pack_bf16x8(acc);
        }
    }
}

// Route-weight gradients of every slot go home: gtw[slot_tk] on the source rank = sum of the partials.
__global__ void __launch_bounds__(256)
droute_push_kernel(const float* droute_part, int n_parts, const int* slot_tk, const int* slot_row, const int* recv_row_base, int S,
                   int N, const uint64_t* arena_ptrs, uint64_t gtw_off) {
    for (int s = blockIdx.x * blockDim.x + threadIdx.x; s < S; s += gridDim.x * blockDim.x) {
        const int tk = slot_tk[s];
        if (tk < 0) continue;
        const int rr = slot_row[s];
        int src = 0;
        while (src + 1 < N && rr >= recv_row_base[src + 1]) ++src;
        float v = 0.f;
        for (int p = 0; p < n_parts; ++p) v += droute_part[(long)s * n_parts + p];
        reinterpret_cast<float*>(arena_ptrs[src] + gtw_off)[tk] = v;
    }
}

// out[0] = max |a-b| ; out[1..5] = sum ab, sum a^2, sum b^2, sum (a+1)(b+1), sum (a+1)^2 + (b+1)^2
__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__global__ void __launch_bounds__(256) numerics_check_kernel(const T* a, const T* b, long n, double* out) {
    double s[5] = {0, 0, 0, 0, 0};
    float mx = 0.f;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        const float x = to_f(a[i]), y = to_f(b[i]);
        mx = fmaxf(mx, fabsf(x - y));
        s[0] += (double)x * y;
        s[1] += (double)x * x;
        s[2] += (double)y * y;
        s[3] += (double)(x + 1.f) * (y + 1.f);
        s[4] += (double)(x + 1.f) * (x + 1.f) + (double)(y + 1.f) * (y + 1.f);
    }
    for (int o = 16; o > 0; o >>= 1) {
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        for (int j = 0; j < 5; ++j) s[j] += __shfl_xor_sync(0xffffffffu, s[j], o);
    }
    if ((threadIdx.x & 31) == 0) {
        atomicMax(reinterpret_cast<unsigned long long*>(out), (unsigned long long)__double_as_longlong((double)mx));
        for (int j = 0; j < 5; ++j) atomicAdd(out + 1 + j, s[j]);
    }
}

int grid_for_warps(long warps, int block) {
    long blocks = (warps * 32 + block - 1) / block;
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 8) blocks = 148 * 8;
    return (int)blocks;
}

}  // namespace

cudaError_t ep_barrier(const uint64_t* signal_ptrs, int rank, int N, int epoch, int* status, int site, int limit_ms, int mode,
                       const int* mask, cudaStream_t stream) {
    const uint64_t limit_ns = limit_ms > 0 ? (uint64_t)limit_ms * 1000000ull : 0ull;   // 0: the status block's run-time limit
    ep_barrier_kernel<<<1, 32 * ((N + 31) / 32), 0, stream>>>(signal_ptrs, rank, N, epoch, status, site, limit_ns, mode, mask);
    return cudaGetLastError();
}

cudaError_t dispatch_push(const void* x, const void* topk_idx, int is64, const float* topk_w, int T, int K, int H, int E, int N,
                          const int* send_slot, const int* send_row, const int* land_off, const uint64_t* arena_ptrs,
                          const SymOffsets& so, int with_meta, int num_blocks, const int* ok, cudaStream_t stream) {
    if (T == 0) return cudaSuccess;
    if (K > 32 || N > 32 || H % 8 != 0) return cudaErrorInvalidValue;
    const int grid = num_blocks > 0 ? num_blocks : grid_for_warps(T, 256);
    dispatch_push_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), topk_idx, is64, topk_w, T, K, H, E, N,
                                                   send_slot, send_row, land_off, arena_ptrs, so, with_meta, ok);
    return cudaGetLastError();
}

cudaError_t tail_fill(void* x, int64_t* idx, float* w, const int* rows_dev, int total_rows, int H, int K, cudaStream_t stream) {
    if (total_rows == 0) return cudaSuccess;
    if (K > 32 || H % 8 != 0) return cudaErrorInvalidValue;
    tail_fill_kernel<<<grid_for_warps(total_rows, 256), 256, 0, stream>>>(static_cast<__nv_bfloat16*>(x), idx, w, rows_dev, total_rows, H, K);
    return cudaGetLastError();
}

cudaError_t expand_rows(const void* rows, const int* slot_row, void* out, int num_slots, int H, cudaStream_t stream) {
    if (num_slots == 0) return cudaSuccess;
    expand_rows_kernel<<<grid_for_warps(num_slots, 256), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(rows), slot_row,
                                                                           static_cast<__nv_bfloat16*>(out), num_slots, H);
    return cudaGetLastError();
}

cudaError_t combine_push(const void* y, const int* row_slots, const int* row_land, const int* recv_row_base, int R, int K, int H,
                         int N, const uint64_t* arena_ptrs, const SymOffsets& so, const float* droute_part, int n_parts,
                         const int* slot_tk, int with_payload, int num_blocks, cudaStream_t stream) {
    if (R == 0) return cudaSuccess;
    const int grid = num_blocks > 0 ? num_blocks : grid_for_warps(R, 256);
    combine_push_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(y), row_slots, row_land, recv_row_base, R, K, H,
                                                  N, arena_ptrs, so, droute_part, n_parts, slot_tk, with_payload);
    return cudaGetLastError();
}

cudaError_t combine_reduce(const void* landing, const int* land_off, const int* ndst, void* out, int T, int H, cudaStream_t stream) {
    if (T == 0) return cudaSuccess;
    combine_reduce_kernel<<<grid_for_warps(T, 256), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(landing), land_off, ndst,
                                                                      static_cast<__nv_bfloat16*>(out), T, H);
    return cudaGetLastError();
}

cudaError_t slot_rows_push(const void* y, const int* slot_tk, const int* slot_row, const int* recv_row_base, int S, int H, int N,
                           const uint64_t* arena_ptrs, uint64_t landing_off, cudaStream_t stream) {
    if (S == 0) return cudaSuccess;
    if (H % 8 != 0) return cudaErrorInvalidValue;
    slot_rows_push_kernel<<<grid_for_warps(S, 256), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(y), slot_tk, slot_row,
                                                                      recv_row_base, S, H, N, arena_ptrs, landing_off);
    return cudaGetLastError();
}

cudaError_t combine_reduce_slots(const void* landing, const void* topk_idx, int is64, void* out, int T, int K, int H, int E,
                                 const float* weights, cudaStream_t stream) {
    if (T == 0) return cudaSuccess;
    if (K > 32 || H % 8 != 0) return cudaErrorInvalidValue;
    combine_reduce_slots_kernel<<<grid_for_warps(T, 256), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(landing), topk_idx, is64,
                                                                            static_cast<__nv_bfloat16*>(out), T, K, H, E, weights);
    return cudaGetLastError();
}

cudaError_t droute_push(const float* droute_part, int n_parts, const int* slot_tk, const int* slot_row, const int* recv_row_base, int S,
                        int N, const uint64_t* arena_ptrs, uint64_t gtw_off, cudaStream_t stream) {
    if (S == 0) return cudaSuccess;
    int blocks = (S + 255) / 256;
    if (blocks > 1184) blocks = 1184;
    droute_push_kernel<<<blocks, 256, 0, stream>>>(droute_part, n_parts, slot_tk, slot_row, recv_row_base, S, N, arena_ptrs, gtw_off);
    return cudaGetLastError();
}

cudaError_t numerics_check(const void* a, const void* b, long n, int is_bf16, double* out6, cudaStream_t stream) {
    cudaError_t e = cudaMemsetAsync(out6, 0, 6 * sizeof(double), stream);
    if (e != cudaSuccess) return e;
    if (n == 0) return cudaSuccess;
    const int grid = (int)((n + 256 * 8 - 1) / (256 * 8) < 1184 ? (n + 256 * 8 - 1) / (256 * 8) : 1184);
    if (is_bf16)
        numerics_check_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(a),
                                                                       static_cast<const __nv_bfloat16*>(b), n, out6);
    else
        numerics_check_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float*>(a), static_cast<const float*>(b), n, out6);
    return cudaGetLastError();
}

}  // namespace tmoe
