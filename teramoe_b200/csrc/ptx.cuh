// Blackwell (sm_100a) PTX primitives used by every kernel in this library:
// mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (UMMA + tensor memory), scoped
// loads/stores for cross-GPU flags, and *bounded* waits.
//
// Every wait in this library has a time limit.  When a limit runs out the waiting
// thread records a status code and returns false; callers unwind to the common
// kernel exit (tensor memory is freed there) and the host turns the status block
// into an exception.  Nothing here traps or spins without a limit.
//
// Role in the reference: csrc/kernels/utils.cuh:69-429 (fences, scoped ld/st,
// mbarrier, bulk copies) and the DeepGEMM/CUTLASS wrappers its GEMM relies on
// (csrc/teramoe/teramoe_wrapper.cuh:532-780).  Its waits trap on timeout
// (csrc/kernels/utils.cuh:518-529); ours return a status instead.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tmoe {

// ---------------------------------------------------------------------------------------------
// Status block (one per rank, in global memory, 8 ints; words 0-3 are zero while all is well).
// word 0: first error code (0 = ok)   word 1: site id   word 2: block index   word 3: detail
// words 4-5: limit in ns (64 bit) of the waits on OTHER ranks (barriers, arrival counters); 0 selects
//            the built-in default.  The host sets it (EPWorld.set_wait_limit_ms), kernels only read it.
// ---------------------------------------------------------------------------------------------
enum StatusCode : int {
    kStatusOk = 0,
    kStatusMbarTimeout = 1,    // an mbarrier phase never completed
    kStatusFlagTimeout = 2,    // a global-memory flag (local or peer) never reached its value
    kStatusBarrierTimeout = 3, // cross-rank barrier did not complete
    kStatusBadArgument = 4,    // device-side consistency check failed (index out of range, ...)
};

__device__ __forceinline__ void report_status(int* status, int code, int site, int detail) {
    if (status == nullptr) return;
    if (atomicCAS(status, 0, code) == 0) {
        status[1] = site;
        status[2] = (int)blockIdx.x;
        status[3] = detail;
        __threadfence_system();
    }
}

// Waits inside one CTA or CTA pair (mbarriers): 2 s is far beyond any healthy pipeline stall.
#ifndef TMOE_WAIT_LIMIT_NS
#define TMOE_WAIT_LIMIT_NS 2000000000ull
#endif
// Waits on another rank see that rank's skew (a checkpoint write, a slow data loader, a first-step build), so
// their limit is a run-time value read from the status block; this is the default when none is set.
// The reference budgets about 100 s for the same waits (csrc/kernels/configs.cuh:20-26).
#ifndef TMOE_PEER_WAIT_LIMIT_NS
#define TMOE_PEER_WAIT_LIMIT_NS 30000000000ull
#endif

__device__ __forceinline__ uint64_t peer_wait_limit_ns(const int* status) {
    if (status == nullptr) return TMOE_PEER_WAIT_LIMIT_NS;
    const uint64_t v = *reinterpret_cast<const volatile uint64_t*>(status + 4);
    return v != 0ull ? v : TMOE_PEER_WAIT_LIMIT_NS;
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() {
    uint32_t l;
    asm volatile("mov.u32 %0, %%laneid;" : "=r"(l));
    return l;
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n"
        " .reg .b32 rx;\n"
        " .reg .pred px;\n"
        " elect.sync rx|px, 0xffffffff;\n"
        " selp.u32 %0, 1, 0, px;\n"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() {
    asm volatile("fence.proxy.async;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        " selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded mbarrier wait.  `abort_flag` is a CTA-shared word: once any role of the CTA gives up it
// is set, and every other wait of the CTA returns false promptly instead of running out its own
// limit.  Returns true when the phase completed.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          int* status, int site) {
#pragma unroll 1
    for (int i = 0; i < 2048; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
#pragma unroll 1
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag != 0u) return false;
        if (globaltimer_ns() - t0 > TMOE_WAIT_LIMIT_NS) {
            *abort_flag = 1u;
            report_status(status, kStatusMbarTimeout, site, (int)parity);
            return false;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// TMA (tiled bulk tensor copies).  The innermost coordinate times the element size must be a
// multiple of 16 bytes; callers in this library only pass multiples of 64 elements of bf16.
// No cluster multicast anywhere: tensor maps may cover memory that peers write into.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
// Row gather: four rows (r.x, r.y, r.z, r.w) of a 2-D tensor, `box[0]` columns starting at column c0,
// land as four consecutive rows in shared memory.  The tensor map must have a box of {cols, 1}.
// Rows that are negative or past the end read as zeros.
__device__ __forceinline__ void tma_gather4(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar, int c0, int4 r) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(r.x), "r"(r.y), "r"(r.z), "r"(r.w)
        : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src_smem, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src_smem), "r"(c0), "r"(c1)
                 : "memory");
}
// Untiled bulk copies: both addresses 16-byte aligned, size a multiple of 16 bytes.  The load completes on
// an mbarrier (complete_tx), the store joins the thread's bulk group.  The global side may be peer memory.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void bulk_store_1d(uint64_t dst, uint32_t src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05: tensor memory + UMMA
// ---------------------------------------------------------------------------------------------
// Allocate `ncols` (power of two, 32..512) tensor-memory columns; the base address is written to
// the shared-memory word `dst_smem`.  Must be executed by one whole warp.
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem], bf16 inputs, fp32 accumulate, one CTA.
__device__ __forceinline__ void umma_bf16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on an mbarrier of this CTA when all previously issued UMMAs have completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---------------------------------------------------------------------------------------------
// CTA pairs (cluster of 2, tcgen05 cta_group::2): one UMMA spans both CTAs' shared and tensor memory.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on an mbarrier of any CTA of the cluster (address from mapa_shared).  Default semantics
// (release at CTA scope): the arrivals of this library publish no data of their own (operand bytes are
// tracked by the TMA transaction count, tensor-memory reads by tcgen05 fences), and a cluster-scope
// release costs a fence of several hundred cycles per arrive, which throttled the whole pipeline.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// The same arrive with a cluster-scope release, for the rare arrive that DOES publish data (a word stored into
// the other CTA's shared memory just before it); pairs with mbar_wait_cluster_acquire.
__device__ __forceinline__ void mbar_arrive_cluster_release(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void st_shared_cluster_u32(uint32_t cluster_addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// Hand 16 bytes to the other CTA of the pair without any fence: the store travels through the async proxy and counts
// 16 bytes on an mbarrier of the destination CTA (like a TMA load does), so a plain wait on that barrier is enough to
// see the data.  `addr` and `bar` are shared::cluster addresses in the same destination CTA.  The barrier also needs one
// arrival that expects the 16 bytes (mbar_arrive_expect_tx_cluster, from this CTA, in either order).
__device__ __forceinline__ void st_async_v4_cluster(uint32_t addr, int4 v, uint32_t bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
                 ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t cluster_bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster_acquire(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
        " selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait with cluster-scope acquire (same contract as mbar_wait).
__device__ __forceinline__ bool mbar_wait_cluster_acquire(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, int* status,
                                                          int site) {
#pragma unroll 1
    for (int i = 0; i < 2048; ++i)
        if (mbar_try_wait_cluster_acquire(bar, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
#pragma unroll 1
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait_cluster_acquire(bar, parity)) return true;
        if (*abort_flag != 0u) return false;
        if (globaltimer_ns() - t0 > TMOE_WAIT_LIMIT_NS) {
            *abort_flag = 1u;
            report_status(status, kStatusMbarTimeout, site, (int)parity);
            return false;
        }
    }
}
__device__ __forceinline__ void tmem_alloc_2cta(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_2cta(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A * B with M = 256 split over the pair (128 rows each) and B's N columns
// split over the pair's shared memory.  Issued by one thread of the pair's first CTA.
__device__ __forceinline__ void umma_bf16_ss_2cta(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                  uint32_t accumulate) {
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on the mbarrier at the same shared-memory offset in every CTA of `cta_mask` once all UMMAs
// issued so far have completed.  (A barrier arrive that is multicast; no data is multicast.)
__device__ __forceinline__ void umma_commit_2cta(uint32_t bar, uint32_t cta_mask) {
    asm volatile(
        "{\n"
        " .reg .b16 lo, hi;\n"
        " mov.b32 {lo, hi}, %1;\n"
        " tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], lo;\n"
        "}\n"
        ::"r"(bar), "r"(cta_mask)
        : "memory");
}
// Tiled load into this CTA's shared memory whose completion bytes are counted on an mbarrier that may
// live in the pair's other CTA (`bar_cluster` from mapa_shared).  The data is not multicast.
__device__ __forceinline__ void tma_load_2d_2cta(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar_cluster, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(c0), "r"(c1)
        : "memory");
}

// Shared-memory matrix descriptor (sm_100 format, version field = 1).
//   start address >> 4 in bits [0,14), leading byte offset >> 4 in [16,30), stride byte offset >> 4
//   in [32,46), version 1 in [46,48), layout type in [61,64) (2 = 128-byte swizzle).
__host__ __device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor for kind::f16 with bf16 A/B and fp32 D.
//   D format (1 = f32) in [4,6), A format (1 = bf16) in [7,10), B format in [10,13),
//   A major in bit 15, B major in bit 16 (0 = K-major, 1 = MN-major), N>>3 in [17,23), M>>4 in [24,29).
__host__ __device__ constexpr uint32_t make_idesc_bf16(uint32_t M, uint32_t N, bool a_mn_major, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
           ((N >> 3) << 17) | ((M >> 4) << 24);
}

// Load 32 consecutive fp32 columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// Scoped global-memory accesses for flags that other SMs or other GPUs write.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int ld_relaxed_sys(const int* p) {
    int v;
    asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_sys(int* p, int v) {
    asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_gpu(int* p, int v) {
    asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }

// 16-byte streaming accesses (payload rows are written once and read once).
__device__ __forceinline__ int4 ld_nc_v4(const void* p) {
    int4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void st_na_v4(void* p, int4 v) {
    asm volatile("st.global.L1::no_allocate.v4.s32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// Warp-wide row copy (nvec 16-byte vectors) with four loads in flight per lane before the stores, so that
// a warp keeps 2 KB outstanding instead of 512 bytes.
__device__ __forceinline__ void warp_copy_row(int4* dst, const int4* src, int nvec, int lane) {
    int i = lane;
    for (; i + 96 < nvec; i += 128) {
        const int4 a = src[i], b = src[i + 32], c = src[i + 64], d = src[i + 96];
        st_na_v4(dst + i, a);
        st_na_v4(dst + i + 32, b);
        st_na_v4(dst + i + 64, c);
        st_na_v4(dst + i + 96, d);
    }
    for (; i < nvec; i += 32) st_na_v4(dst + i, src[i]);
}

// Bounded wait until *flag >= target (acquire, system scope).  One thread calls it.
// limit_ns == 0: the run-time limit for waits on other ranks (status block words 4-5, else the default).
__device__ __forceinline__ bool wait_flag_ge_sys(const int* flag, int target, int* status, int site, uint64_t limit_ns = 0ull) {
    if (ld_acquire_sys(flag) >= target) return true;
    if (limit_ns == 0ull) limit_ns = peer_wait_limit_ns(status);
    const uint64_t t0 = globaltimer_ns();
#pragma unroll 1
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i) {
            if (ld_acquire_sys(flag) >= target) return true;
            __nanosleep(64);
        }
        if (status != nullptr && ld_relaxed_sys(status) != 0) return false;  // someone else already gave up
        if (globaltimer_ns() - t0 > limit_ns) {
            report_status(status, kStatusFlagTimeout, site, target);
            return false;
        }
    }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
    __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
    return __bfloat1622float2(v);
}

}  // namespace tmoe
