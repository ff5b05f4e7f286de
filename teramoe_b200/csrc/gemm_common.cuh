// Shared pieces of the tcgen05 grouped GEMM kernels (gemm.cu: one CTA per tile; gemm2.cu: CTA pairs):
// tile constants, the argument block, the epilogue math and the host-side tensor-map helpers.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mutex>

#include "ptx.cuh"

namespace tmoe {
namespace detail {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UK = 16;
constexpr int kStages = 4;
constexpr int kAStageBytes = BM * BK * 2;  // 16 KB
constexpr int kBStageBytes = BN * BK * 2;  // 32 KB
constexpr int kStageBytes = kAStageBytes + kBStageBytes;
constexpr int kAtomBytes = 64 * BK * 2;  // one 64(MN) x 64(K) MN-major swizzle atom column: 8 KB
constexpr int kEpiWarps = 8;
constexpr int kThreads = 128 + 32 * kEpiWarps;
constexpr int kTmemCols = 512;
constexpr int kSuperM = 16;  // m-blocks per L2 super-group
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;

enum Epilogue : int { kEpiStore = 0, kEpiSwiGLU = 1, kEpiDSwiGLU = 2, kEpiPush = 3 };

struct GemmArgs {
    int n_total;                 // columns of D per group
    int k_total;                 // K of the M-grouped modes
    int num_n_blocks;            // ceil(n_total / BN)
    int max_mblocks;             // static bound on m-blocks (M-grouped) or ceil(m_total / BM) (K-grouped)
    const int* num_mblocks_dev;  // optional device-side live count (M-grouped)
    const int* mblock_expert;    // [max_mblocks] expert of each m-block (M-grouped)
    int b_group_rows;            // rows of the B tensor map per expert
    int num_groups;              // K-grouped: number of experts
    const int* seg_offsets;      // K-grouped: [num_groups + 1] row offsets, multiples of 128
    int m_total;                 // K-grouped: rows of dW per expert
    int kgroup_n_fast;           // K-grouped, CTA pairs: consecutive tiles walk the column blocks first (else the row units)
    __nv_bfloat16* d;            // main output
    int ldd;
    __nv_bfloat16* aux;          // preact (fwd gate_up) / dGU (bwd grad_act)
    int ld_aux;
    const __nv_bfloat16* preact; // bwd grad_act input
    const float* row_w;          // route weight per slot row
    const int* unit_blk;         // CTA-pair kernels: [max_units + 1] first m-block of each unit (last = block count)
    const int* num_units_dev;    // CTA-pair kernels: device-side live unit count
    int max_units;               // CTA-pair kernels: bound on units (M-grouped); unused in weight-gradient mode
    // kEpiPush: every output row goes straight to the rank that owns the token (peer store over NVLink):
    // row s lands at push_ptrs[source rank of s] + push_off + slot_tk[s] * ldd elements.
    const unsigned long long* push_ptrs;  // [ranks] base address of every rank's symmetric arena
    unsigned long long push_off;          // byte offset of the per-(token,k) landing table inside the arena
    const int* slot_tk;                   // [rows] t*K+k of the row's entry at its source (-1 = pad row)
    const int* slot_row;                  // [rows] receive row (locates the source rank through recv_row_base)
    const int* recv_row_base;             // [ranks+1]
    int num_ranks;
    // Backward push (whole-layer kernel only): with gtw_off != 0 the tiles of the first column block also send the
    // row's route-weight gradient (sum of droute_part[row, :]) to gtw[slot_tk[row]] of the token's rank.
    unsigned long long gtw_off;
    const float* droute_in;
    int n_parts_in;
    const int* gather_rows;      // GATHER modes: source row of each slot-space row (-1 = zero row)
    float* droute_part;          // bwd grad_act: [rows, n_parts]
    int n_parts;
    int* status;
};

struct Tile {
    int m_blk, n_blk, group, k0, nk;  // k0: first K row (elements), nk: number of BK blocks
};

template <bool KGROUP>
__device__ __forceinline__ bool get_tile(const GemmArgs& g, int t, int num_mblocks, Tile& tile) {
    if constexpr (!KGROUP) {
        const int total = num_mblocks * g.num_n_blocks;
        if (t >= total) return false;
        const int per_super = kSuperM * g.num_n_blocks;
        const int super = t / per_super;
        const int r = t - super * per_super;
        const int m_first = super * kSuperM;
        const int m_cnt = min(kSuperM, num_mblocks - m_first);
        tile.n_blk = r / m_cnt;
        tile.m_blk = m_first + (r - tile.n_blk * m_cnt);
        tile.group = g.mblock_expert[tile.m_blk];
        tile.k0 = 0;
        tile.nk = g.k_total / BK;
        return true;
    } else {
        const int per_group = g.max_mblocks * g.num_n_blocks;
        const int total = g.num_groups * per_group;
        if (t >= total) return false;
        tile.group = t / per_group;
        const int r = t - tile.group * per_group;
        tile.n_blk = r / g.max_mblocks;
        tile.m_blk = r - tile.n_blk * g.max_mblocks;
        const int s0 = g.seg_offsets[tile.group];
        const int s1 = g.seg_offsets[tile.group + 1];
        tile.k0 = s0;
        tile.nk = (s1 - s0) / BK;
        return true;
    }
}

__device__ __forceinline__ void store_bf16x8(__nv_bfloat16* p, const uint32_t* acc) {
    int4 v;
    v.x = (int)pack_bf16x2(__uint_as_float(acc[0]), __uint_as_float(acc[1]));
    v.y = (int)pack_bf16x2(__uint_as_float(acc[2]), __uint_as_float(acc[3]));
    v.z = (int)pack_bf16x2(__uint_as_float(acc[4]), __uint_as_float(acc[5]));
    v.w = (int)pack_bf16x2(__uint_as_float(acc[6]), __uint_as_float(acc[7]));
    *reinterpret_cast<int4*>(p) = v;
}

// One epilogue thread: its TMEM lane (= tile row) and 128 accumulator columns starting at taddr0 /
// global column n0.  Converts, applies the fused element-wise math and stores.
template <int EPI>
__device__ __forceinline__ void epilogue_thread(const GemmArgs& g, uint32_t taddr0, long row, bool row_ok, int n0, int part_idx,
                                                bool zero_tile) {
    float w = 0.f;
    if constexpr (EPI == kEpiSwiGLU || EPI == kEpiDSwiGLU) w = g.row_w[row];
    __nv_bfloat16* push_dst = nullptr;
    if constexpr (EPI == kEpiPush) {
        const int tk = row_ok ? g.slot_tk[row] : -1;
        if (tk < 0) {
            row_ok = false;
        } else {
            const int rr = g.slot_row[row];
            int src = 0;
            while (src + 1 < g.num_ranks && rr >= g.recv_row_base[src + 1]) ++src;
            push_dst = reinterpret_cast<__nv_bfloat16*>(g.push_ptrs[src] + g.push_off) + (long)tk * g.ldd;
        }
    }
    float droute = 0.f;
#pragma unroll 1
    for (int c = 0; c < (BN / 2) / 32; ++c) {
        const int col = n0 + c * 32;
        int4 pre[8];
        if constexpr (EPI == kEpiDSwiGLU) {
            // issue the pre-activation loads before the tensor-memory load so their latencies overlap
            if (col < g.n_total) {
                const int4* pp = reinterpret_cast<const int4*>(g.preact + row * (2l * g.n_total) + 2 * col);
#pragma unroll
                for (int v = 0; v < 8; ++v) pre[v] = ld_nc_v4(pp + v);
            }
        }
        uint32_t acc[32];
        tmem_ld_x32(taddr0 + (uint32_t)(c * 32), acc);
        tmem_ld_wait();
        if (zero_tile) {
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = 0u;
        }
        if constexpr (EPI == kEpiStore || EPI == kEpiPush) {
            if (row_ok) {
                __nv_bfloat16* dst = (EPI == kEpiPush ? push_dst : g.d + row * g.ldd) + col;
#pragma unroll
                for (int v = 0; v < 4; ++v)
                    if (col + v * 8 + 8 <= g.n_total) store_bf16x8(dst + v * 8, acc + v * 8);
            }
        } else if constexpr (EPI == kEpiSwiGLU) {
            // accumulator columns (2j, 2j+1) = (gate_j, up_j); n_total = 2I
            if (col < g.n_total) {
                store_bf16x8(g.aux + row * g.ld_aux + col, acc);
                store_bf16x8(g.aux + row * g.ld_aux + col + 8, acc + 8);
                store_bf16x8(g.aux + row * g.ld_aux + col + 16, acc + 16);
                store_bf16x8(g.aux + row * g.ld_aux + col + 24, acc + 24);
                uint32_t o[8];
#pragma unroll
                for (int p = 0; p < 8; ++p) {
                    float a2[2];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float gt = __uint_as_float(acc[4 * p + 2 * e]);
                        const float up = __uint_as_float(acc[4 * p + 2 * e + 1]);
                        a2[e] = __fdividef(gt, 1.f + __expf(-gt)) * up * w;
                    }
                    o[p] = pack_bf16x2(a2[0], a2[1]);
                }
                __nv_bfloat16* dst = g.d + row * g.ldd + (col >> 1);
                *reinterpret_cast<int4*>(dst) = make_int4((int)o[0], (int)o[1], (int)o[2], (int)o[3]);
                *reinterpret_cast<int4*>(dst + 8) = make_int4((int)o[4], (int)o[5], (int)o[6], (int)o[7]);
            }
        } else {
            // accumulator column j = d act_j; n_total = I.  preact holds (g_j, u_j) at [2j, 2j+1].
            if (col < g.n_total) {
                uint32_t dgu[32];
                uint32_t aw[16];
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                    const int4 pv = pre[v];
                    const uint32_t pr[4] = {(uint32_t)pv.x, (uint32_t)pv.y, (uint32_t)pv.z, (uint32_t)pv.w};
                    float av[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 gu = unpack_bf16x2(pr[e]);
                        const float ga = __uint_as_float(acc[4 * v + e]);
                        const float sig = __fdividef(1.f, 1.f + __expf(-gu.x));
                        const float s = gu.x * sig;
                        const float a = s * gu.y;
                        const float gaw = ga * w;
                        const float d_up = s * gaw;
                        const float d_gate = (sig - s * sig + s) * gaw * gu.y;
                        dgu[4 * v + e] = pack_bf16x2(d_gate, d_up);
                        av[e] = a * w;
                        droute += ga * a;
                    }
                    aw[2 * v] = pack_bf16x2(av[0], av[1]);
                    aw[2 * v + 1] = pack_bf16x2(av[2], av[3]);
                }
                int4* dg = reinterpret_cast<int4*>(g.aux + row * g.ld_aux + 2 * col);
#pragma unroll
                for (int v = 0; v < 8; ++v)
                    dg[v] = make_int4((int)dgu[4 * v], (int)dgu[4 * v + 1], (int)dgu[4 * v + 2], (int)dgu[4 * v + 3]);
                int4* da = reinterpret_cast<int4*>(g.d + row * g.ldd + col);
#pragma unroll
                for (int v = 0; v < 4; ++v)
                    da[v] = make_int4((int)aw[4 * v], (int)aw[4 * v + 1], (int)aw[4 * v + 2], (int)aw[4 * v + 3]);
            }
        }
    }
    if constexpr (EPI == kEpiDSwiGLU) g.droute_part[row * g.n_parts + part_idx] = droute;
}

// ---------------------------------------------------------------------------------------------
// Push epilogue (combine fused into the GEMM): an epilogue warp's 32 rows x 128 columns leave for the ranks that
// own the tokens.  Each lane stages its row in shared memory 64 columns (128 bytes) at a time and hands the segment
// to a bulk copy shared -> peer global, so no thread of the epilogue waits for NVLink: the warp goes straight back
// to draining tensor memory, and only re-using the staging row waits until the copy engine has READ it
// (cp.async.bulk.wait_group.read), not until the peer has the bytes.  The caller ends with tma_store_wait<0>()
// before the kernel exits or before it tells anyone that the rows are there.
// ---------------------------------------------------------------------------------------------
constexpr int kPushRowBytes = 128 + 16;                        // 64 bf16 columns + pad (bank-conflict-free rows, 16-byte aligned)
constexpr int kPushWarpBytes = 32 * kPushRowBytes;             // one epilogue warp stages 32 rows x 64 columns

// Address of the landing row of output row `row` (0 for pad rows and for rows of a block that is not live).
__device__ __forceinline__ unsigned long long push_row_address(const GemmArgs& g, long row, bool live, int* src_rank) {
    if (!live) return 0ull;
    const int tk = g.slot_tk[row];
    if (tk < 0) return 0ull;
    const int rr = g.slot_row[row];
    int src = 0;
    while (src + 1 < g.num_ranks && rr >= g.recv_row_base[src + 1]) ++src;
    if (src_rank != nullptr) *src_rank = src;
    return g.push_ptrs[src] + g.push_off + (unsigned long long)tk * g.ldd * 2ull;
}

// taddr0: this warp's tensor-memory lanes and first accumulator column; n0: global column of taddr0;
// my_row_smem: this lane's staging row (kPushRowBytes apart between lanes).
__device__ __forceinline__ void push_epilogue_warp(const GemmArgs& g, uint32_t taddr0, unsigned long long dst_row, int n0,
                                                   uint32_t my_row_smem) {
#pragma unroll 1
    for (int cg = 0; cg < 2; ++cg) {
        tma_store_wait_read<0>();          // this lane's previous segment has left shared memory
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {
            uint32_t acc[32];
            tmem_ld_x32(taddr0 + (uint32_t)(cg * 64 + c2 * 32), acc);
            tmem_ld_wait();
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const uint32_t p0 = pack_bf16x2(__uint_as_float(acc[8 * v]), __uint_as_float(acc[8 * v + 1]));
                const uint32_t p1 = pack_bf16x2(__uint_as_float(acc[8 * v + 2]), __uint_as_float(acc[8 * v + 3]));
                const uint32_t p2 = pack_bf16x2(__uint_as_float(acc[8 * v + 4]), __uint_as_float(acc[8 * v + 5]));
                const uint32_t p3 = pack_bf16x2(__uint_as_float(acc[8 * v + 6]), __uint_as_float(acc[8 * v + 7]));
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(my_row_smem + (uint32_t)(c2 * 64 + v * 16)),
                             "r"(p0), "r"(p1), "r"(p2), "r"(p3) : "memory");
            }
        }
        const int col0 = n0 + cg * 64;
        if (dst_row != 0ull && col0 + 64 <= g.n_total) {
            fence_proxy_async_smem();      // this lane's generic-proxy stores -> the bulk copy's read
            bulk_store_1d(dst_row + (unsigned long long)col0 * 2ull, my_row_smem, 128u);
        }
        tma_store_commit();
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// 2-D bf16 row-major tensor [rows, cols] (cols contiguous), box {box_cols, box_rows}, 128-byte swizzle.
inline cudaError_t make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_cols, uint32_t box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (fn == nullptr) return cudaErrorNotSupported;
    if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (cols * 2) % 16 != 0) return cudaErrorInvalidValue;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// The dynamic shared-memory limit of a kernel is a per-device attribute: set it once on every device that launches it.
template <typename Kernel>
inline cudaError_t ensure_smem_limit(Kernel kern, int bytes, bool (&done)[64]) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64 && done[dev]) return cudaSuccess;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess && dev >= 0 && dev < 64) done[dev] = true;
    return e;
}

inline int default_sms(int num_sms) {
    if (num_sms > 0) return num_sms;
    static int cached = 0;
    if (cached == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, dev);
    }
    return cached;
}



// CTA-pair launchers (gemm2.cu).  kind: 0 gate_up+SwiGLU, 1 down, 2 grad_act+dSwiGLU, 3 dX.
}  // namespace detail
cudaError_t gemm2_mgroup(int kind, const void* a, const void* b, const detail::GemmArgs& g, int a_rows, int a_cols, int b_rows,
                         int b_cols, int num_sms, cudaStream_t stream);
cudaError_t gemm2_wgrad(const void* a, const void* b, const detail::GemmArgs& g, int rows, int M, int N, int num_sms,
                        cudaStream_t stream);
}  // namespace tmoe
